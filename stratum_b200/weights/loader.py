"""Binding weights by tensor name, with one error that says everything that is wrong.

The reference looks each tensor up by its formatted name and reports a missing
one (stratum/native/stratum_arch_llama.inc.c:595-634, FIND / FIND_OPTIONAL);
its safetensors resolver checks dtype and rank (stratum/native/stratum_st.h:370-393).
Here the model's parts declare every tensor they expect (name, shape, role);
the loader compares that list with what the files hold and raises a single
`WeightError` listing missing tensors, unexpected tensors and wrong shapes.

Dtype policy: a "matrix" is kept in the compute dtype (bfloat16 stays bfloat16 on
the bfloat16 path; it is widened, exactly, on the float32 path); a "vector"
(gain, bias) is held in float32, which is exact from bfloat16; "keep" tensors
stay in the dtype the file stores (a float32 tensor stays float32); "index"
tables become int32.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Sequence

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files


class WeightError(ValueError):
    """The model folder's tensors do not match what the model expects."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{where}: weights do not match the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def check_tensors(where: str, expected: Mapping[str, TensorSpec], present: Mapping[str, object],
                  ignored_suffixes: Sequence[str] = ()) -> None:
    """`present`: name -> object with .shape and .dtype.  Raises WeightError if they disagree.
    ignored_suffixes: names ending in one of these are no weights of the model and may be present."""
    missing = [n for n, s in expected.items() if n not in present and not s.optional]
    unexpected = [n for n in present if n not in expected and not n.endswith(tuple(ignored_suffixes) or ("\0",))]
    wrong = []
    for n, s in expected.items():
        if n not in present:
            continue
        e = present[n]
        if tuple(e.shape) != tuple(s.shape):
            wrong.append(f"{n}: file has {list(e.shape)}, model needs {list(s.shape)}")
        elif s.role == "index" and e.dtype not in _INTS:
            wrong.append(f"{n}: file has {e.dtype}, model needs an integer table")
        elif s.role != "index" and e.dtype not in _FLOATS:
            wrong.append(f"{n}: file has {e.dtype}, model needs floating point")
    if missing or unexpected or wrong:
        raise WeightError(where, sorted(missing), sorted(unexpected), wrong)


def place(t: torch.Tensor, spec: TensorSpec, compute_dtype: torch.dtype, device) -> torch.Tensor:
    """Copy one tensor to the device in the dtype its role asks for."""
    if spec.role == "index":
        dt = torch.int32
    elif spec.role == "vector":
        dt = torch.float32
    elif spec.role == "keep":
        dt = t.dtype if t.dtype in (torch.float32, torch.bfloat16) else torch.float32
    else:
        dt = compute_dtype
    if t.dtype == dt:
        return t.to(device, copy=True).contiguous()
    # widen or narrow on the device: one pass over the data, no float32 staging copy on the host
    return t.to(device).to(dt).contiguous()


def load_weights(model_dir: str, expected: Mapping[str, TensorSpec], compute_dtype: torch.dtype,
                 device, ignored_suffixes: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Read every expected tensor of a model folder onto the device."""
    files = open_model_files(model_dir)
    try:
        present = {}
        owner: Dict[str, SafetensorsFile] = {}
        for f in files:
            for n, e in f.entries.items():
                if n in present:
                    raise SafetensorsError(f"{model_dir}: tensor {n!r} appears in two shards")
                present[n] = e
                owner[n] = f
        check_tensors(model_dir, expected, present, ignored_suffixes)
        out = {}
        for n, s in expected.items():
            if n in present:
                out[n] = place(owner[n].tensor(n), s, compute_dtype, device)
        return out
    finally:
        for f in files:
            f.close()
