"""Plain, slow restatement of the Llama dense decoder, used only as a test oracle.

Whole sequences, no cache, one function per part, no code shared with the
product package.  Every function cites the reference formula it restates
(paths are relative to the reference project root, shiaho777/stratum).

Rests on the reference's formulas; the interleaved-RoPE, bias-free, untied
subset is additionally pinned once against the reference's own PyTorch oracle
(stratum/tools/hidden_oracle.py) by tests/golden/make_golden.py.

Precision: everything is computed in float64 from the given weights, so the
oracle sits at the exact value of the formulas; the reference itself keeps
float32 values with float64 sums (RMSNorm, softmax denominator), which lies
within float32 rounding of this.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np

F64 = np.float64


def _as_f32(a: np.ndarray) -> np.ndarray:
    """Round to float32 and return as float64."""
    return np.asarray(a, dtype=np.float32).astype(F64)


# --------------------------------------------------------------------------- parts

def embed(table: np.ndarray, token_ids: Sequence[int]) -> np.ndarray:
    """x = E[token]: a row gather without scaling.
    stratum/native/stratum_arch_llama.inc.c:564-593, :702."""
    return np.asarray(table, dtype=F64)[np.asarray(token_ids, dtype=np.int64)]


def rms_norm(x: np.ndarray, gain: np.ndarray, eps: float) -> np.ndarray:
    """y = x * (1/sqrt(mean(x^2) + eps)) * gain.
    stratum/native/stratum_arch_llama.inc.c:45-76 (sum of squares in double,
    scale = 1/sqrt(ss/N + eps))."""
    x = np.asarray(x, dtype=F64)
    ss = np.sum(x * x, axis=-1, keepdims=True)
    scale = 1.0 / np.sqrt(ss / x.shape[-1] + F64(eps))
    return x * scale * np.asarray(gain, dtype=F64)


def head_rms_norm(heads: np.ndarray, gain: np.ndarray, eps: float) -> np.ndarray:
    """RMSNorm of every head on its own, [T, n_heads, head_dim] with a gain of head_dim values: the optional
    norm of queries and keys, applied after the projection and before the rotation.
    stratum/native/stratum_arch_llama.inc.c:403-420 (one token), :866-884 (a chunk)."""
    return np.stack([rms_norm(heads[:, j], gain, eps) for j in range(heads.shape[1])], axis=1)


def linear(x: np.ndarray, weight: np.ndarray, bias: Optional[np.ndarray] = None) -> np.ndarray:
    """y[r] = sum_k W[r][k] * x[k] (+ b[r]); W is row-major [out][in].
    stratum/native/stratum_linear.h:491-507 (no bias there); the bias form
    y = b + W x is stratum/native/stratum_algo.h:36-54."""
    y = np.asarray(x, dtype=F64) @ np.asarray(weight, dtype=F64).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=F64)
    return y


def rope_inv_freq(rope_dim: int, theta: float, scaling: Optional[dict] = None) -> np.ndarray:
    """inv_k = 1 / theta^(2k / rope_dim), k < rope_dim/2.
    stratum/native/stratum_arch_llama.inc.c:114-129, stratum/native/stratum_rope.h:82-86.

    scaling (keys as in a Llama config.json `rope_scaling`):
      linear: inv_k / factor                      (stratum/native/stratum_rope.h:87-88)
      llama3: wavelength-dependent blend of inv_k and inv_k/factor.  This rule
              is not in the reference; it is the published Llama-3.1 rule:
              lambda = 2*pi/inv_k;  lambda < orig/high -> inv_k;
              lambda > orig/low -> inv_k/factor;  otherwise
              s = (orig/lambda - low)/(high - low), inv = (1-s)*inv_k/factor + s*inv_k.
    """
    n_pairs = rope_dim // 2
    k = np.arange(n_pairs, dtype=F64)
    inv = 1.0 / (F64(theta) ** (2.0 * k / F64(rope_dim)))
    inv = _as_f32(inv)          # the reference keeps the table in float32 (powf)
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind in ("default", "none", None):
        return inv
    factor = F64(scaling["factor"])
    if kind == "linear":
        return _as_f32(inv / factor)
    if kind == "llama3":
        low = F64(scaling["low_freq_factor"])
        high = F64(scaling["high_freq_factor"])
        orig = F64(scaling["original_max_position_embeddings"])
        out = np.empty_like(inv)
        for i, f in enumerate(inv):
            lam = 2.0 * math.pi / f
            if lam < orig / high:
                out[i] = f
            elif lam > orig / low:
                out[i] = f / factor
            else:
                s = (orig / lam - low) / (high - low)
                out[i] = (1.0 - s) * f / factor + s * f
        return _as_f32(out)
    if kind == "yarn":
        # stratum/native/stratum_rope.h:76-106: a ramp over the pair index between the plain frequency (pairs that
        # turn more than beta_fast times within the original context) and the interpolated one (fewer than beta_slow)
        if not factor > 1.0:
            return inv
        orig = F64(scaling["original_max_position_embeddings"])
        dim = F64(rope_dim)

        def corr_dim(n_rot):                    # stratum/native/stratum_rope.h:76-79
            return dim * math.log(orig / (F64(n_rot) * 2.0 * math.pi)) / (2.0 * math.log(F64(theta)))

        low = max(0.0, math.floor(corr_dim(scaling.get("beta_fast", 32.0))))
        high = min(dim - 1.0, math.ceil(corr_dim(scaling.get("beta_slow", 1.0))))
        denom = max(high - low, 0.001)
        out = np.empty_like(inv)
        for i, f in enumerate(inv):
            ramp = 1.0 - min(1.0, max(0.0, (i - low) / denom))
            out[i] = (f / factor) * (1.0 - ramp) + f * ramp
        return _as_f32(out)
    raise ValueError(f"plain oracle: unknown rope scaling {kind!r}")


def rope_magnitude(scaling: Optional[dict]) -> float:
    """The factor on cos and sin: 1 except for yarn, where it is attention_factor if that is
    positive and 0.1 ln(factor) + 1 otherwise.  stratum/native/stratum_rope.h:108-112."""
    if not scaling or scaling.get("rope_type", scaling.get("type")) != "yarn" or not scaling["factor"] > 1.0:
        return 1.0
    att = scaling.get("attention_factor", -1.0)
    return float(att) if att is not None and att > 0 else 0.1 * math.log(float(scaling["factor"])) + 1.0


def apply_rope(x: np.ndarray, positions: np.ndarray, inv_freq: np.ndarray,
               interleaved: bool, magnitude: float = 1.0) -> np.ndarray:
    """Rotate pairs of one head vector by angle = pos * inv_k.
    x: [T, n_heads, head_dim]; dims >= 2*len(inv_freq) are left untouched.
    interleaved pairs (2k, 2k+1): stratum/native/stratum_arch_llama.inc.c:149-156;
    half-split pairs (k, k + n_pairs): stratum/native/stratum_arch_llama.inc.c:139-147.
    (x0, x1) <- (x0*c - x1*s, x0*s + x1*c); cos and sin are multiplied by `magnitude`
    (stratum/native/stratum_arch_llama.inc.c:143, :152), so only rotated components grow."""
    x = np.array(x, dtype=F64, copy=True)
    n_pairs = inv_freq.shape[0]
    # angle = (float)pos * inv_k in float32, as the reference computes it (:141, :151)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * inv_freq.astype(np.float32)[None, :]).astype(F64)
    c = np.cos(ang)[:, None, :] * F64(magnitude)
    s = np.sin(ang)[:, None, :] * F64(magnitude)
    if interleaved:
        i0 = np.arange(n_pairs) * 2
        i1 = i0 + 1
    else:
        i0 = np.arange(n_pairs)
        i1 = i0 + n_pairs
    x0 = x[..., i0].copy()
    x1 = x[..., i1].copy()
    x[..., i0] = x0 * c - x1 * s
    x[..., i1] = x0 * s + x1 * c
    return x


def softmax(scores: np.ndarray) -> np.ndarray:
    """p = exp(s - max) / sum.  stratum/native/stratum_engine.h:395-423."""
    m = np.max(scores, axis=-1, keepdims=True)
    e = np.exp(scores - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def causal_gqa_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray,
                         window: int = 0) -> np.ndarray:
    """q: [T, Nq, Hd], k/v: [T, Nk, Hd] (already rotated) -> [T, Nq, Hd].
    score_t = (q_h . K_t[kv(h)]) / sqrt(Hd), kv(h) = h // (Nq/Nk); only keys
    t <= own position are visited; softmax; o = sum_t p_t V_t.
    stratum/native/stratum_arch_llama.inc.c:435, :444, :467-514.
    window > 0 keeps only the last `window` keys (not used by Llama)."""
    T, Nq, Hd = q.shape
    Nk = k.shape[1]
    gs = Nq // Nk
    scale = 1.0 / math.sqrt(Hd)
    out = np.zeros((T, Nq, Hd), dtype=F64)
    for i in range(T):
        lo = 0 if window <= 0 else max(0, i - window + 1)
        for h in range(Nq):
            kv = h // gs
            s = (k[lo:i + 1, kv, :] @ q[i, h, :]) * scale
            p = softmax(s)
            out[i, h, :] = p @ v[lo:i + 1, kv, :]
    return out


def silu(z: np.ndarray) -> np.ndarray:
    """silu(z) = z / (1 + exp(-z)).  stratum/native/stratum_engine.h:373-391."""
    return z / (1.0 + np.exp(-z))


def swiglu_mlp(xn: np.ndarray, w: Dict[str, np.ndarray], prefix: str) -> np.ndarray:
    """down(silu(gate(xn)) * up(xn)).  stratum/native/stratum_arch_llama.inc.c:550-555."""
    g = linear(xn, w[prefix + "gate_proj.weight"], w.get(prefix + "gate_proj.bias"))
    u = linear(xn, w[prefix + "up_proj.weight"], w.get(prefix + "up_proj.bias"))
    return linear(silu(g) * u, w[prefix + "down_proj.weight"], w.get(prefix + "down_proj.bias"))


def attention_block(xn: np.ndarray, positions: np.ndarray, w: Dict[str, np.ndarray], prefix: str,
                    cfg: dict, inv_freq: np.ndarray) -> np.ndarray:
    """q,k,v projections, RoPE on q and k, causal GQA attention, output projection.
    stratum/native/stratum_arch_llama.inc.c:398-524."""
    T = xn.shape[0]
    Nq, Nk, Hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = linear(xn, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).reshape(T, Nq, Hd)
    k = linear(xn, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).reshape(T, Nk, Hd)
    v = linear(xn, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).reshape(T, Nk, Hd)
    inter = bool(cfg.get("rope_interleaved", False))
    mag = rope_magnitude(cfg.get("rope_scaling"))
    q = apply_rope(q, positions, inv_freq, inter, mag)
    k = apply_rope(k, positions, inv_freq, inter, mag)
    o = causal_gqa_attention(q, k, v).reshape(T, Nq * Hd)
    return linear(o, w[prefix + "o_proj.weight"], w.get(prefix + "o_proj.bias"))


def decoder_layer(x: np.ndarray, positions: np.ndarray, w: Dict[str, np.ndarray], li: int,
                  cfg: dict, inv_freq: np.ndarray) -> np.ndarray:
    """x += attn(norm(x)); x += mlp(norm(x)).
    stratum/native/stratum_arch_llama.inc.c:392-396, :524-532, :555."""
    p = f"model.layers.{li}."
    eps = cfg["rms_norm_eps"]
    xn = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(xn, positions, w, p + "self_attn.", cfg, inv_freq)
    xn = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(xn, w, p + "mlp.")
    return x


# --------------------------------------------------------------------------- whole model

def normalized_config(cfg: dict) -> dict:
    """Fill the defaults a Llama config.json may leave out."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("tie_word_embeddings", False)
    return c


def forward_hidden(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int],
                   capture_layers: Sequence[int] = ()) -> (np.ndarray, Dict[int, np.ndarray]):
    """Residual stream after the last layer for a whole sequence, [T, H];
    also the residual after each layer in capture_layers.
    stratum/native/stratum_arch_llama.inc.c:688-716."""
    c = normalized_config(cfg)
    positions = np.arange(len(tokens))
    inv_freq = rope_inv_freq(int(c.get("rope_dim") or c["head_dim"]), c["rope_theta"],
                             c.get("rope_scaling"))
    x = embed(w["model.embed_tokens.weight"], tokens)
    caps = {}
    for li in range(c["num_hidden_layers"]):
        x = decoder_layer(x, positions, w, li, c, inv_freq)
        if li in capture_layers:
            caps[li] = x.copy()
    return x, caps


def forward_logits(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    """Logits at every position of one whole sequence, [T, V] float64.
    Final norm then the output head; the head is lm_head.weight if present,
    else the embedding table (tied).  stratum/native/stratum_arch_llama.inc.c:713-723."""
    c = normalized_config(cfg)
    x, _ = forward_hidden(c, w, tokens)
    xn = rms_norm(x, w["model.norm.weight"], c["rms_norm_eps"])
    head = w.get("lm_head.weight")
    if head is None:
        head = w["model.embed_tokens.weight"]
    return linear(xn, head)


def argmax_lowest(logits: np.ndarray) -> int:
    """Index of the maximum; the lowest index wins ties.
    stratum/native/stratum_engine.h:429-463."""
    best, mv = 0, logits[0]
    for i in range(1, logits.shape[0]):
        if logits[i] > mv:
            best, mv = i, logits[i]
    return int(best)


def greedy_generate(cfg: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], n_new: int,
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """Greedy continuation by re-running the whole sequence for every token.
    stratum/native/stratum_arch_llama.inc.c:1611, :2041-2061."""
    seq = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        nxt = argmax_lowest(forward_logits(cfg, w, seq)[-1])
        out.append(nxt)
        seq.append(nxt)
        if nxt in stop_ids:
            break
    return out


# --------------------------------------------------------------------------- sampling oracle

class Pcg32:
    """PCG32 stream as the reference seeds and steps it.
    stratum/native/stratum_arch_qwen35.inc.c:13973-13992 (state/inc, seeding),
    :13990-13992 (uniform = (u32 >> 8) * 2^-24),
    :14010-14018 (stream s uses seed + s * 0x9E3779B97F4A7C15)."""
    MULT = 6364136223846793005
    MASK = (1 << 64) - 1

    def __init__(self, seed: int, stream: int = 0):
        seed = (seed + stream * 0x9E3779B97F4A7C15) & self.MASK
        self.state = 0
        self.inc = ((seed << 1) | 1) & self.MASK
        self.next_u32()
        self.state = (self.state + 0x853C49E6748FEA9B) & self.MASK
        self.next_u32()

    def next_u32(self) -> int:
        old = self.state
        self.state = (old * self.MULT + self.inc) & self.MASK
        xorshifted = (((old >> 18) ^ old) >> 27) & 0xFFFFFFFF
        rot = old >> 59
        return ((xorshifted >> rot) | (xorshifted << ((-rot) & 31))) & 0xFFFFFFFF

    def uniform(self) -> float:
        return float(np.float32(self.next_u32() >> 8) * np.float32(1.0 / 16777216.0))


def temperature_probs(logits: np.ndarray, temp: float) -> np.ndarray:
    """p_i = exp((l_i - max)/T) / sum.  stratum/native/stratum_arch_qwen35.inc.c:14069-14080."""
    l = np.asarray(logits, dtype=F64)
    e = np.exp((l - l.max()) / F64(temp))
    return e / e.sum()


def filtered_distribution(logits: np.ndarray, temp: float, top_k: int, top_p: float):
    """Candidate ids and probabilities after temperature, top-k and top-p, in the order
    the draw walks them: by descending probability (lower id first among equals)
    when a filter is on, by id otherwise.
    stratum/native/stratum_arch_qwen35.inc.c:14034-14099."""
    p = temperature_probs(logits, temp)
    ids = np.arange(p.shape[0])
    if top_k <= 0 and top_p >= 1.0:
        return ids, p
    order = np.lexsort((ids, -np.asarray(logits, dtype=F64)))   # descending logit, then id
    if top_k > 0:
        order = order[:top_k]
    pp = p[order] / p[order].sum()
    if top_p < 1.0:
        cum = np.cumsum(pp)
        keep = int(np.searchsorted(cum, top_p, side="left")) + 1
        keep = min(keep, pp.shape[0])
        order, pp = order[:keep], pp[:keep]
        pp = pp / pp.sum()
    return order, pp


def sample_inverse_cdf(ids: np.ndarray, probs: np.ndarray, u: float) -> int:
    """First candidate with u < cumulative probability; the last one if none.
    stratum/native/stratum_arch_qwen35.inc.c:14101-14109."""
    cum = 0.0
    for i, p in zip(ids, probs):
        cum += p
        if u < cum:
            return int(i)
    return int(ids[-1])
