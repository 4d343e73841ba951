"""A plain, slow implementation of the Llama forward pass and the sampler in numpy.

It rests on the reference's formulas, one function for each part, whole sequences, no
cache, and it shares no code with the package under test: it has its own safetensors
reader, its own rotary table, its own exp.  Every float32 operation is rounded the way
the reference's C++ rounds it (``-ffp-contract=off``: a product and a sum are two
roundings unless the reference writes ``std::fma``), so that in float32 it reproduces the
reference bit for bit.  ``fma32`` emulates a fused multiply-add exactly through float64
with round-to-odd.

Two switches:
  * ``exp``: ``"libm"`` calls glibc's expf as the reference does (src/kernels.cpp:296,326);
    ``"det"`` is the reproducible exp that the CUDA kernels use (same operations in the
    same order; constants given as bit patterns).
  * ``round_bf16``: rounds activations to bfloat16 at the places where the bfloat16
    engine stores them (after a norm, after a projection, after rotation, the softmax
    weights before the value product, the attention output, the SwiGLU output).  The
    reference has no such path (its activations are always float32, src/model.h:75); this
    mode exists to compare the bfloat16 kernels with a tight tolerance.
"""
from __future__ import annotations

import ctypes
import json
import os
import struct

import numpy as np

f32 = np.float32
_libm = ctypes.CDLL("libm.so.6")
for _n in ("expf", "cosf", "sinf"):
    getattr(_libm, _n).restype = ctypes.c_float
    getattr(_libm, _n).argtypes = [ctypes.c_float]
_libm.powf.restype = ctypes.c_float
_libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
_libm.fmaf.restype = ctypes.c_float
_libm.fmaf.argtypes = [ctypes.c_float] * 3


def _libm_map(fn, x):
    x = np.asarray(x, dtype=f32)
    flat = x.reshape(-1)
    out = np.empty_like(flat)
    for i in range(flat.size):
        out[i] = fn(float(flat[i]))
    return out.reshape(x.shape)


# --------------------------------------------------------------------------------------
# exact float32 arithmetic helpers

def fma32(a, b, c):
    """round_to_float32(a * b + c) with a single rounding, elementwise.

    a * b is exact in float64 (24 + 24 bits).  The float64 sum is rounded to odd (if it
    was inexact and its last bit is even, step one unit towards the true value), after
    which the conversion to float32 rounds correctly (Boldo and Melquiond).
    """
    a = np.asarray(a, dtype=f32).astype(np.float64)
    b = np.asarray(b, dtype=f32).astype(np.float64)
    c = np.asarray(c, dtype=f32).astype(np.float64)
    p = a * b
    s = p + c
    bb = s - p
    err = (p - (s - bb)) + (c - bb)
    s, err = np.broadcast_arrays(s, err)
    s = np.array(s, dtype=np.float64)
    bits = s.view(np.int64)
    inexact = err != 0.0
    even = (bits & 1) == 0
    fix = inexact & even
    # towards the true value: up in magnitude if err has the sign of s, else down
    up = (err > 0) == (s > 0)
    step = np.where(up, 1, -1).astype(np.int64)
    bits += np.where(fix, step, 0)
    return s.astype(f32)


def bf16_round(x):
    """float32 -> nearest bfloat16 (ties to even) -> float32 (src/model.cpp:69-74)."""
    x = np.ascontiguousarray(x, dtype=f32)
    b = x.view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFFFFFF
    return ((b >> 16) << 16).astype(np.uint32).view(f32).reshape(x.shape)


def _bits(h):
    return np.array([h], dtype=np.uint32).view(f32)[0]


def exp_det(x):
    """The reproducible exp of the CUDA kernels, operation for operation."""
    x = np.asarray(x, dtype=f32)
    xc = np.clip(x, f32(-87.0), f32(88.0))
    t = xc * _bits(0x3fb8aa3b)
    magic = _bits(0x4b400000)
    n = (t + magic) - magic
    r = fma32(n, _bits(0xbf318000), xc)
    r = fma32(n, _bits(0x395e8083), r)
    p = np.full_like(r, _bits(0x39506967))
    for c in (0x3ab743ce, 0x3c088908, 0x3d2aa9c1, 0x3e2aaaaa, 0x3f000000):
        p = fma32(p, r, _bits(c))
    z = r * r
    y = fma32(p, z, r)
    y = y + f32(1.0)
    scale = ((n.astype(np.int32) + 127) << 23).astype(np.uint32).view(f32)
    out = (y * scale).astype(f32)
    out = np.where(x < f32(-87.0), f32(0.0), out)
    out = np.where(x > f32(88.0), f32(np.inf), out)
    return out.astype(f32)


def exp_libm(x):
    return _libm_map(_libm.expf, x)


EXP = {"libm": exp_libm, "det": exp_det}


# --------------------------------------------------------------------------------------
# parts

def dot16(a, b):
    """Canonical dot product over the last axis (src/kernels.cpp:57-64,86-100): 16
    lane-wise fused chains, lane = i % 16, then s8[i] = l[i] + l[i+8], s4[i] = s8[i] +
    s8[i+4], (s4[0] + s4[2]) + (s4[1] + s4[3])."""
    a = np.asarray(a, dtype=f32)
    b = np.asarray(b, dtype=f32)
    a, b = np.broadcast_arrays(a, b)
    n = a.shape[-1]
    lanes = np.zeros(a.shape[:-1] + (16,), dtype=f32)
    for i in range(0, n, 16):
        w = min(16, n - i)
        lanes[..., :w] = fma32(a[..., i:i + w], b[..., i:i + w], lanes[..., :w])
    s8 = lanes[..., :8] + lanes[..., 8:]
    s4 = s8[..., :4] + s8[..., 4:]
    return ((s4[..., 0] + s4[..., 2]) + (s4[..., 1] + s4[..., 3])).astype(f32)


def rmsnorm(x, w, eps):
    """y = (x * inv) * w with inv = 1 / sqrt(dot16(x, x) / dim + eps) (src/kernels.cpp:264-271)."""
    x = np.asarray(x, dtype=f32)
    dim = x.shape[-1]
    ss = dot16(x, x)
    inv = f32(1.0) / np.sqrt(ss / f32(dim) + f32(eps), dtype=f32)
    return ((x * inv[..., None]).astype(f32) * np.asarray(w, dtype=f32)).astype(f32)


def linear(x, W):
    """y[m][n] = one fused chain over k ascending of x[m][k] * W[n][k] (src/kernels.cpp:236-244)."""
    x = np.asarray(x, dtype=f32)
    W = np.asarray(W, dtype=f32)
    acc = np.zeros((x.shape[0], W.shape[0]), dtype=f32)
    for k in range(x.shape[1]):
        acc = fma32(x[:, k:k + 1], W[None, :, k], acc)
    return acc


def rope_inv_freq(head_dim, theta, scaling=None):
    """inv_freq[i] = 1.0f / powf(theta, (float)(2i) / (float)hd) (src/model.cpp:220-225).

    ``scaling`` = dict of the llama3 rule (not in the reference, which rejects any
    rope_scaling, tools/convert.py:59-60): with wavelen = 2*pi / inv_freq, frequencies
    with wavelen < orig/high stay, those with wavelen > orig/low are divided by factor,
    the band between is blended linearly in (orig/wavelen - low) / (high - low); computed
    in float64 from the float32 base value and rounded once to float32."""
    half = head_dim // 2
    inv = np.empty(half, dtype=f32)
    for i in range(half):
        e = f32(f32(2 * i) / f32(head_dim))
        inv[i] = f32(1.0) / f32(_libm.powf(float(f32(theta)), float(e)))
    if scaling:
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        out = np.empty(half, dtype=f32)
        for i in range(half):
            fr = float(inv[i])
            wavelen = 2.0 * np.pi / fr
            if wavelen < orig / high:
                v = fr
            elif wavelen > orig / low:
                v = fr / factor
            else:
                smooth = (orig / wavelen - low) / (high - low)
                v = (1.0 - smooth) * fr / factor + smooth * fr
            out[i] = f32(v)
        inv = out
    return inv


def rope(v, positions, inv_freq):
    """Rotate-half pairs (i, i + hd/2): angle = (float)pos * inv_freq[i]; cosf / sinf;
    v[i] = x1*c - x2*s, v[i+hd/2] = x2*c + x1*s, each product rounded on its own
    (src/kernels.cpp:273-289).  v: [T, heads, hd]."""
    v = np.asarray(v, dtype=f32)
    half = v.shape[-1] // 2
    ang = (np.asarray(positions, dtype=f32)[:, None] * inv_freq[None, :]).astype(f32)
    c = _libm_map(_libm.cosf, ang)[:, None, :]
    s = _libm_map(_libm.sinf, ang)[:, None, :]
    x1, x2 = v[..., :half], v[..., half:]
    o1 = ((x1 * c).astype(f32) - (x2 * s).astype(f32)).astype(f32)
    o2 = ((x2 * c).astype(f32) + (x1 * s).astype(f32)).astype(f32)
    return np.concatenate([o1, o2], axis=-1)


def attention(q, k, v, exp="libm", window=0, round_bf16=False):
    """Causal attention of one whole sequence (src/kernels.cpp:312-338,342-368).

    q: [T, heads, hd], k, v: [T, kv_heads, hd].  Head h uses kv head h // (heads/kv_heads).
    Pass 1: s_j = dot16(q, k_j) * scale for j = lo..t (scale = 1/sqrtf(hd), applied after
    the dot), mx = max.  Pass 2, j ascending: e = exp(s_j - mx); sum += e;
    acc[d] = fma(e, v_j[d], acc[d]).  o = acc * (1 / sum).  ``window`` > 0 keeps only the
    last ``window`` keys (the reference has no window)."""
    expf = EXP[exp]
    T, heads, hd = q.shape
    kvh = k.shape[1]
    grp = heads // kvh
    scale = f32(1.0) / np.sqrt(f32(hd), dtype=f32)
    kk = np.repeat(k, grp, axis=1)  # [T, heads, hd]
    vv = np.repeat(v, grp, axis=1)
    out = np.empty((T, heads, hd), dtype=f32)
    # Query rows are taken in blocks only to bound the memory of the broadcast below; a row's
    # arithmetic does not depend on the block it is in.
    for t0 in range(0, T, 32):
        t1 = min(T, t0 + 32)
        R, J = t1 - t0, t1  # rows of the block, keys 0 .. t1-1
        # scores[t, h, j]
        s = dot16(q[t0:t1, :, None, :], np.transpose(kk[:J], (1, 0, 2))[None, :, :, :])
        s = (s * scale).astype(f32)
        t_idx = np.arange(t0, t1)[:, None, None]
        j_idx = np.arange(J)[None, None, :]
        valid = j_idx <= t_idx
        if window and window > 0:
            valid &= j_idx > t_idx - window
        mx = np.max(np.where(valid, s, f32(-np.inf)), axis=2, keepdims=True)
        e = np.where(valid, expf(np.where(valid, s - mx, f32(0.0)).astype(f32)), f32(0.0)).astype(f32)
        e_pv = bf16_round(e) if round_bf16 else e
        ssum = np.zeros((R, heads), dtype=f32)
        acc = np.zeros((R, heads, hd), dtype=f32)
        for j in range(J):
            m = np.broadcast_to(valid[:, :, j], (R, heads))
            ssum = np.where(m, (ssum + e[:, :, j]).astype(f32), ssum)
            upd = fma32(e_pv[:, :, j, None], vv[j][None, :, :], acc)
            acc = np.where(m[:, :, None], upd, acc)
        inv = (f32(1.0) / ssum).astype(f32)
        out[t0:t1] = (acc * inv[:, :, None]).astype(f32)
    return out


def swiglu(gate_up, inter, exp="libm"):
    """h = g * (1 / (1 + exp(-g))) * u, left to right, rows laid out [gate | up]
    (src/kernels.cpp:291-298)."""
    g = np.asarray(gate_up[:, :inter], dtype=f32)
    u = np.asarray(gate_up[:, inter:], dtype=f32)
    sig = (f32(1.0) / (f32(1.0) + EXP[exp]((-g).astype(f32))).astype(f32)).astype(f32)
    return ((g * sig).astype(f32) * u).astype(f32)


# --------------------------------------------------------------------------------------
# model folder -> arrays (own reader of the safetensors layout, tools/convert.py:41-50)

def read_safetensors(path):
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        if info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(f32)
        elif info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(f32)
        else:
            raise ValueError("plain reader: dtype " + info["dtype"])
        out[name] = a.reshape(info["shape"])
    return out


class PlainLlama:
    """Whole-sequence forward of the decoder of src/model.cpp:267-322, one sequence at a time."""

    def __init__(self, folder, exp="libm", round_bf16=False, window=0):
        with open(os.path.join(folder, "config.json")) as f:
            c = json.load(f)
        self.c = c
        self.exp = exp
        self.round_bf16 = round_bf16
        self.window = window
        self.hidden = c["hidden_size"]
        self.layers = c["num_hidden_layers"]
        self.heads = c["num_attention_heads"]
        self.kv_heads = c.get("num_key_value_heads", self.heads)
        self.hd = c.get("head_dim") or self.hidden // self.heads
        self.inter = c["intermediate_size"]
        self.vocab = c["vocab_size"]
        self.eps = c.get("rms_norm_eps", 1e-6)
        self.tied = c.get("tie_word_embeddings", False)
        self.inv_freq = rope_inv_freq(self.hd, c.get("rope_theta", 10000.0), c.get("rope_scaling"))
        self.w = {}
        for fn in sorted(os.listdir(folder)):
            if fn.endswith(".safetensors"):
                self.w.update(read_safetensors(os.path.join(folder, fn)))
        if round_bf16:  # the bfloat16 engine holds its matrices in bfloat16
            for n in list(self.w):
                if self.w[n].ndim == 2:
                    self.w[n] = bf16_round(self.w[n])

    def _r(self, x):
        return bf16_round(x) if self.round_bf16 else x

    def logits(self, tokens, start=0):
        """Logits [T, vocab] at every position of one sequence."""
        w, L = self.w, "model.layers.%d."
        T = len(tokens)
        pos = np.arange(start, start + T)
        x = w["model.embed_tokens.weight"][np.asarray(tokens)].astype(f32)  # src/model.cpp:274
        for l in range(self.layers):
            p = L % l
            xn = self._r(rmsnorm(x, w[p + "input_layernorm.weight"], self.eps))          # model.cpp:281
            q = self._r(linear(xn, w[p + "self_attn.q_proj.weight"]))                    # model.cpp:282
            k = self._r(linear(xn, w[p + "self_attn.k_proj.weight"]))
            v = self._r(linear(xn, w[p + "self_attn.v_proj.weight"]))
            q = self._r(rope(q.reshape(T, self.heads, self.hd), pos, self.inv_freq))      # model.cpp:289
            k = self._r(rope(k.reshape(T, self.kv_heads, self.hd), pos, self.inv_freq))   # model.cpp:290
            v = v.reshape(T, self.kv_heads, self.hd)
            a = attention(q, k, v, self.exp, self.window, self.round_bf16)                # model.cpp:298
            a = self._r(a).reshape(T, self.heads * self.hd)
            x = (x + linear(a, w[p + "self_attn.o_proj.weight"])).astype(f32)            # model.cpp:299-300
            xn = self._r(rmsnorm(x, w[p + "post_attention_layernorm.weight"], self.eps))  # model.cpp:301
            gu = np.concatenate([linear(xn, w[p + "mlp.gate_proj.weight"]),
                                 linear(xn, w[p + "mlp.up_proj.weight"])], axis=1)        # model.cpp:302
            h = self._r(swiglu(self._r(gu), self.inter, self.exp))                        # model.cpp:303
            x = (x + linear(h, w[p + "mlp.down_proj.weight"])).astype(f32)               # model.cpp:304-305
        xn = self._r(rmsnorm(x, w["model.norm.weight"], self.eps))                        # model.cpp:318
        head = w["model.embed_tokens.weight"] if self.tied else w["lm_head.weight"]       # model.cpp:170-171
        return linear(xn, head)                                                            # model.cpp:319-320


# --------------------------------------------------------------------------------------
# sampler (src/engine.cpp:12-16,31-80)

_MASK = (1 << 64) - 1


def mix64(z):
    z &= _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def counter_uniform(seed, position, stream=0):
    """u in [0, 1), a pure function of (seed, position, stream) (src/engine.cpp:35-38)."""
    z = mix64(mix64((seed ^ 0x6A09E667F3BCC909) & _MASK) ^ mix64((position * 4 + stream) & _MASK))
    return float(z >> 11) * 2.0 ** -53


def argmax_row(logits):
    """First index of the maximum (src/engine.cpp:40-45)."""
    best = 0
    for i in range(1, len(logits)):
        if logits[i] > logits[best]:
            best = i
    return best


def sample_row(logits, temperature, u, exp="libm"):
    """w_i = expf((l_i - mx) / T) in float32; total and cumulative sums in float64 in
    vocabulary order; the first i with cum > u * total, skipping w_i <= 0, else the last
    positive i (src/engine.cpp:50-80)."""
    l = np.asarray(logits, dtype=f32)
    mx = np.max(l)
    w = EXP[exp](((l - mx).astype(f32) / f32(temperature)).astype(f32))
    total = 0.0
    for x in w:
        total += float(x)
    target = u * total
    cum, last = 0.0, 0
    for i, x in enumerate(w):
        if x <= 0.0:
            continue
        cum += float(x)
        last = i
        if cum > target:
            return last
    return last


def fingerprint(h, logits_row):
    """Chained hash of the raw bits of a logits row (src/engine.cpp:18-29)."""
    data = np.ascontiguousarray(logits_row, dtype=f32).tobytes()
    i = 0
    while i + 8 <= len(data):
        (wd,) = struct.unpack_from("<Q", data, i)
        h = ((h ^ wd) * 1099511628211) & _MASK
        i += 8
    while i < len(data):
        h = ((h ^ data[i]) * 1099511628211) & _MASK
        i += 1
    return mix64(h)


def generate(model, prompt, max_new_tokens, temperature=0.0, seed=0, eos_id=-1, ignore_eos=False,
             exp=None):
    """Greedy / temperature generation by whole-sequence recomputation; the sampler is keyed
    by the position the new token will occupy (src/engine.cpp:470-476)."""
    exp = exp or model.exp
    toks = list(prompt)
    out = []
    fp = 1469598103934665603
    for _ in range(max_new_tokens):
        row = model.logits(toks)[-1]
        if temperature <= 0:
            t = argmax_row(row)
        else:
            t = sample_row(row, temperature, counter_uniform(seed, len(toks), 0), exp)
        fp = fingerprint(fp, row)
        toks.append(int(t))
        out.append(int(t))
        if not ignore_eos and t == eos_id:
            break
    return out, fp
