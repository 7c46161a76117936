#!/usr/bin/env python3
"""Pin the plain oracle's rotation frequencies on the reference's own C code.

The reference's header for rotary frequencies (stratum/native/stratum_rope.h) is plain C and compiles with
gcc on any CPU.  This script writes a driver of a dozen lines that includes that header, evaluates
`stratum_rope_inv_freq` for every pair and `stratum_rope_mscale` for a few parameter sets (no scaling,
linear, YaRN with and without an explicit attention factor), compiles and runs it, and stores what it prints
in tests/golden/rope_reference.json.  tests/test_plain_reference.py compares tests/plain/llama_plain.py's
`rope_inv_freq` and `rope_magnitude` with that file.  (llama3 scaling is not in the reference, so nothing of
the reference can pin it; it rests on its formula, stated in the oracle's docstring.)

Usage:  python tests/golden/make_rope_golden.py --reference /path/to/reference/checkout
"""
import argparse
import json
import os
import subprocess
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, type 0 none / 1 linear / 2 yarn, theta, factor, attn_factor (<0 derive), beta_fast, beta_slow, orig_ctx, pairs)
CASES = [
    ("none_64", 0, 10000.0, 1.0, -1.0, 32.0, 1.0, 0, 32),
    ("linear_f2_48", 1, 1000.0, 2.0, -1.0, 32.0, 1.0, 0, 24),
    ("yarn_f4_orig32_80", 2, 50000.0, 4.0, -1.0, 4.0, 0.5, 32, 40),
    ("yarn_f8_orig4096_128", 2, 500000.0, 8.0, -1.0, 32.0, 1.0, 4096, 64),
    ("yarn_f4_attn1.25_64", 2, 10000.0, 4.0, 1.25, 32.0, 1.0, 2048, 32),
]

DRIVER = r'''
#include "stratum_rope.h"
int main(void) {
%s
    return 0;
}
'''

ONE = r'''    {
        StratumRope r; stratum_rope_defaults(&r, (float)%(theta).9g);
        r.type = %(type)d; r.factor = (float)%(factor).9g; r.attn_factor = (float)%(attn).9g;
        r.beta_fast = (float)%(bf).9g; r.beta_slow = (float)%(bs).9g; r.orig_ctx = %(orig)d;
        printf("%(name)s %%.9g", stratum_rope_mscale(&r));
        for (int k = 0; k < %(pairs)d; k++) printf(" %%.9g", stratum_rope_inv_freq(&r, k, %(pairs)d));
        printf("\n");
    }
'''


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("STRATUM_REFERENCE"))
    args = ap.parse_args()
    if not args.reference:
        ap.error("give --reference DIR (a checkout of shiaho777/stratum) or set STRATUM_REFERENCE")
    native = os.path.join(args.reference, "stratum", "native")
    body = "".join(ONE % dict(name=n, type=t, theta=th, factor=f, attn=a, bf=bf, bs=bs, orig=o, pairs=p)
                   for n, t, th, f, a, bf, bs, o, p in CASES)
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = os.path.join(tmp, "rope_driver.c"), os.path.join(tmp, "rope_driver")
        with open(src, "w") as fh:
            fh.write(DRIVER % body)
        subprocess.run(["gcc", "-O1", "-std=c11", "-I", native, src, "-o", exe, "-lm"], check=True)
        text = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    out = {}
    for line, case in zip(text.strip().splitlines(), CASES):
        name, mscale, *freqs = line.split()
        assert name == case[0] and len(freqs) == case[8]
        out[name] = {"type": ["none", "linear", "yarn"][case[1]], "theta": case[2], "factor": case[3],
                     "attention_factor": case[4], "beta_fast": case[5], "beta_slow": case[6],
                     "original_max_position": case[7], "pairs": case[8], "mscale": float(mscale),
                     "inv_freq": [float(x) for x in freqs]}
    dst = os.path.join(HERE, "rope_reference.json")
    with open(dst, "w") as fh:
        json.dump(out, fh, indent=1)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
