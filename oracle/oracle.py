"""CPU oracle for the fused-MoE hot path: loader for the C restatement plus an independent
numpy restatement and the seeded input generator.

TEST INFRASTRUCTURE ONLY.  The shipped package never imports this module; only tests, the
smoke check and the benchmark's CPU-baseline / reference arm do.

PARITY UNPINNED: the reference project (TheRock) only declares a build of Composable
Kernel (math-libs/CMakeLists.txt:553-620) whose source lives in an empty submodule
(.gitmodules:19-22).  No reference source, golden vector or test exists for this path, so
the arithmetic contract is the one written at the top of fmoe_oracle.c.  The numpy
functions below restate that contract a second time, with different loop structure, so the
two can be checked against each other.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfmoe_oracle.so")
_lib = None

QUANT_NONE, QUANT_TOKEN_CHANNEL, QUANT_BLOCK128, QUANT_BLOCK128_UE8M0 = 0, 1, 2, 3


def build(force: bool = False) -> str:
    """Compile fmoe_oracle.c with the committed Makefile (gcc, OpenMP)."""
    src = os.path.join(_HERE, "fmoe_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_sort_capacity.restype = ctypes.c_int64
        _lib.orc_sort_capacity.argtypes = [ctypes.c_int64] * 4
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


# ---------------------------------------------------------------------------- RNG
# Counter-based generator (Philox4x32-10 + Box-Muller) so inputs depend only on
# (seed, stream, element index), never on generation order or library version.

_PHILOX_M0 = np.uint64(0xD2511F53)
_PHILOX_M1 = np.uint64(0xCD9E8D57)
_PHILOX_W0 = 0x9E3779B9
_PHILOX_W1 = 0xBB67AE85


def philox4x32(counter: np.ndarray, seed: int, stream: int) -> np.ndarray:
    """counter: uint64 [n] -> uint32 [n,4]."""
    c0 = (counter & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    c1 = (counter >> np.uint64(32)).astype(np.uint64)
    c2 = np.full_like(c0, np.uint64(stream & 0xFFFFFFFF))
    c3 = np.zeros_like(c0)
    k0 = seed & 0xFFFFFFFF
    k1 = (seed >> 32) & 0xFFFFFFFF
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = _PHILOX_M0 * c0
        p1 = _PHILOX_M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        n0 = hi1 ^ c1 ^ np.uint64(k0)
        n2 = hi0 ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0, lo1, n2, lo0
        k0 = (k0 + _PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def normal(shape, seed: int, stream: int, std: float = 1.0) -> np.ndarray:
    """N(0, std^2) f32 tensor; element i uses Philox block i//4, lane i%4."""
    n = int(np.prod(shape))
    nb = (n + 3) // 4
    out = np.empty(nb * 4, dtype=np.float32)
    chunk = 1 << 22
    for b0 in range(0, nb, chunk):
        b1 = min(nb, b0 + chunk)
        r = philox4x32(np.arange(b0, b1, dtype=np.uint64), seed, stream)
        u = (r.astype(np.float64) + 0.5) * (1.0 / 4294967296.0)
        rad0 = np.sqrt(-2.0 * np.log(u[:, 0]))
        rad1 = np.sqrt(-2.0 * np.log(u[:, 2]))
        z = np.stack([rad0 * np.cos(2 * np.pi * u[:, 1]), rad0 * np.sin(2 * np.pi * u[:, 1]),
                      rad1 * np.cos(2 * np.pi * u[:, 3]), rad1 * np.sin(2 * np.pi * u[:, 3])], axis=1)
        out[b0 * 4:b1 * 4] = (z.reshape(-1) * std).astype(np.float32)
    return out[:n].reshape(shape)


# ---------------------------------------------------------------------------- formats

def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(a), _p(out), ctypes.c_int64(a.size))
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_e4m3(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint8)
    lib().orc_f32_to_e4m3(_p(a), _p(out), ctypes.c_int64(a.size))
    return out


def e4m3_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint8)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_e4m3_to_f32(_p(a), _p(out), ctypes.c_int64(a.size))
    return out


def quant_rows_e4m3(a: np.ndarray, group: int | None = None, pow2: bool = False):
    """[rows, cols] f32 -> (e4m3 bytes [rows, cols], scales [rows, cols/group]); pow2: scales
    rounded up to powers of two."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    rows, cols = a.shape
    group = cols if group is None else group
    q = np.empty((rows, cols), dtype=np.uint8)
    s = np.empty((rows, cols // group), dtype=np.float32)
    lib().orc_quant_rows_e4m3_ex(_p(a), ctypes.c_int64(rows), ctypes.c_int64(cols),
                                 ctypes.c_int64(group), 1 if pow2 else 0, _p(q), _p(s))
    return q, s


def quant_blocks_e4m3(a: np.ndarray, pow2: bool = False):
    """[rows, cols] f32 -> (e4m3 bytes, scales [rows/128, cols/128])."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    rows, cols = a.shape
    q = np.empty((rows, cols), dtype=np.uint8)
    s = np.empty((rows // 128, cols // 128), dtype=np.float32)
    lib().orc_quant_blocks_e4m3_ex(_p(a), ctypes.c_int64(rows), ctypes.c_int64(cols), 1 if pow2 else 0, _p(q), _p(s))
    return q, s


# ---------------------------------------------------------------------------- C oracle

def route(logits: np.ndarray, K: int, mode: str = "softmax"):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    T, E = logits.shape
    ids = np.empty((T, K), dtype=np.int32)
    w = np.empty((T, K), dtype=np.float32)
    rc = lib().orc_route(_p(logits), T, E, K, 0 if mode == "softmax" else 1, _p(ids), _p(w))
    if rc != 0:
        raise ValueError(f"orc_route failed: {rc}")
    return ids, w


def sort_capacity(T: int, K: int, E: int, block_m: int) -> int:
    return int(lib().orc_sort_capacity(T, K, E, block_m))


def moe_sorting(topk_ids: np.ndarray, topk_w: np.ndarray, E: int, block_m: int):
    """Returns dict(sorted_token_ids, sorted_weights, sorted_rows, sorted_expert_ids,
    num_tokens_post_pad, mblk_cum)."""
    topk_ids = np.ascontiguousarray(topk_ids, dtype=np.int32)
    topk_w = np.ascontiguousarray(topk_w, dtype=np.float32)
    T, K = topk_ids.shape
    cap = sort_capacity(T, K, E, block_m)
    out = dict(
        sorted_token_ids=np.empty(cap, np.int32), sorted_weights=np.empty(cap, np.float32),
        sorted_rows=np.empty(cap, np.int32), sorted_expert_ids=np.empty(cap // block_m, np.int32),
        num_tokens_post_pad=np.empty(1, np.int32), mblk_cum=np.empty(E + 1, np.int32))
    lib().orc_moe_sorting(_p(topk_ids), _p(topk_w), T, K, E, block_m,
                          _p(out["sorted_token_ids"]), _p(out["sorted_weights"]),
                          _p(out["sorted_rows"]), _p(out["sorted_expert_ids"]),
                          _p(out["num_tokens_post_pad"]), _p(out["mblk_cum"]))
    return out


def fused_moe(x_bf16, w1, w2, topk_ids, topk_w, quant=QUANT_NONE, w1_scale=None, w2_scale=None,
              sel=None, n_threads: int = 0, gate_only: bool = False, partial_bf16: bool = False) -> np.ndarray:
    """x_bf16 [T,H] uint16; w1 [E,2I,H], w2 [E,H,I] (uint16 bf16 bits or uint8 e4m3 bytes).
    Returns out [n_sel or T, H] as bf16 bits (uint16)."""
    x_bf16 = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    wdt = np.uint16 if quant == QUANT_NONE else np.uint8
    w1 = np.ascontiguousarray(w1, dtype=wdt)
    w2 = np.ascontiguousarray(w2, dtype=wdt)
    topk_ids = np.ascontiguousarray(topk_ids, dtype=np.int32)
    topk_w = np.ascontiguousarray(topk_w, dtype=np.float32)
    T, H = x_bf16.shape
    E, I2, H2 = w1.shape
    I = I2 if gate_only else I2 // 2
    assert H2 == H and w2.shape == (E, H, I)
    K = topk_ids.shape[1]
    if w1_scale is not None:
        w1_scale = np.ascontiguousarray(w1_scale, dtype=np.float32)
        w2_scale = np.ascontiguousarray(w2_scale, dtype=np.float32)
    if sel is not None:
        sel = np.ascontiguousarray(sel, dtype=np.int32)
    n = T if sel is None else len(sel)
    out = np.empty((n, H), dtype=np.uint16)
    rc = lib().orc_fused_moe_ex2(T, H, I, E, K, quant, 1 if gate_only else 0, 1 if partial_bf16 else 0,
                                 _p(x_bf16), _p(w1), _p(w2),
                                _p(w1_scale), _p(w2_scale), _p(topk_ids), _p(topk_w), _p(sel),
                                0 if sel is None else len(sel), _p(out), n_threads)
    if rc != 0:
        raise ValueError(f"orc_fused_moe failed: {rc}")
    return out


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---------------------------------------------------------------------------- numpy restatement
# Written independently of the C code (vectorised matmuls instead of per-row dot loops).

def np_f32_to_bf16(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> np.uint64(16)) & np.uint64(1)
    r = (u + np.uint64(0x7FFF) + lsb) >> np.uint64(16)
    return r.astype(np.uint16)


def np_e4m3_table() -> np.ndarray:
    b = np.arange(256)
    s, e, m = b >> 7, (b >> 3) & 15, b & 7
    v = np.where(e == 0, m * 2.0 ** -9, (1 + m / 8.0) * 2.0 ** (e.astype(np.float64) - 7))
    v = np.where((e == 15) & (m == 7), np.nan, v)
    return np.where(s == 1, -v, v).astype(np.float32)


def np_f32_to_e4m3(a: np.ndarray) -> np.ndarray:
    """Nearest-even onto the e4m3 grid by searching the sorted table of finite values."""
    tab = np_e4m3_table()
    pos = tab[:127].astype(np.float64)          # 0 .. 448, ascending, codes 0..126
    x = np.ascontiguousarray(a, dtype=np.float32).astype(np.float64)
    sign = np.signbit(x)
    ax = np.minimum(np.abs(x), 448.0)
    hi = np.clip(np.searchsorted(pos, ax, side="left"), 0, 126)
    lo = np.clip(hi - 1, 0, 126)
    dlo, dhi = ax - pos[lo], pos[hi] - ax
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    return np.where(sign, code | 0x80, code).astype(np.uint8)


def np_pow2_ceil(t: np.ndarray) -> np.ndarray:
    """Smallest power of two >= t (t > 0, f32), exponent clamped to [-126, 127]."""
    m, e = np.frexp(t.astype(np.float64))            # t = m * 2^e, m in [0.5, 1)
    e = np.where(m == 0.5, e - 1, e)
    return np.ldexp(1.0, np.clip(e, -126, 127)).astype(np.float32)


def np_quant(a: np.ndarray, group: int, pow2: bool = False):
    rows, cols = a.shape
    g = a.reshape(rows, cols // group, group).astype(np.float32)
    amax = np.abs(g).max(axis=2)
    s = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    if pow2:
        s = np.where(amax > 0, np_pow2_ceil(s), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / s).astype(np.float32)
    q = np_f32_to_e4m3((g * inv[:, :, None]).astype(np.float32))
    return q.reshape(rows, cols), s


def np_route(logits: np.ndarray, K: int, mode: str = "softmax"):
    l = logits.astype(np.float32)
    if mode == "softmax":
        ex = np.exp(l - l.max(axis=1, keepdims=True), dtype=np.float32)
        s = ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)
    else:
        s = (np.float32(1) / (np.float32(1) + np.exp(-l, dtype=np.float32))).astype(np.float32)
    ids = np.argsort(-s, axis=1, kind="stable")[:, :K].astype(np.int32)
    w = np.take_along_axis(s, ids, axis=1)
    return ids, (w / w.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)


def np_moe_sorting(topk_ids: np.ndarray, topk_w: np.ndarray, E: int, block_m: int):
    T, K = topk_ids.shape
    flat = topk_ids.reshape(-1)
    cap = (T * K + E * (block_m - 1) + block_m - 1) // block_m * block_m
    tok = np.full(cap, T, np.int32)
    wts = np.zeros(cap, np.float32)
    rows = np.full(cap, -1, np.int32)
    eids = np.full(cap // block_m, -1, np.int32)
    cum = np.zeros(E + 1, np.int32)
    pos = 0
    for e in range(E):
        idx = np.nonzero(flat == e)[0]
        n = len(idx)
        tok[pos:pos + n] = idx // K
        wts[pos:pos + n] = topk_w.reshape(-1)[idx]
        rows[pos:pos + n] = idx
        nb = -(-n // block_m)
        eids[pos // block_m:pos // block_m + nb] = e
        pos += nb * block_m
        cum[e + 1] = pos // block_m
    return dict(sorted_token_ids=tok, sorted_weights=wts, sorted_rows=rows, sorted_expert_ids=eids,
                num_tokens_post_pad=np.array([pos], np.int32), mblk_cum=cum)


def np_fused_moe(x_bf16, w1, w2, topk_ids, topk_w, quant=QUANT_NONE, w1_scale=None, w2_scale=None,
                 gate_only: bool = False, partial_bf16: bool = False):
    """Per-expert batched restatement (float32 matmuls).  Same contract as orc_fused_moe;
    summation order inside the dot products differs, so agreement is to f32 round-off."""
    T, H = x_bf16.shape
    E, I2, _ = w1.shape
    I = I2 if gate_only else I2 // 2
    K = topk_ids.shape[1]
    x = bf16_to_f32(x_bf16)
    tab = np_e4m3_table()
    slots = np.zeros((T, K, H), np.float32)
    for e in range(E):
        t_idx, k_idx = np.nonzero(topk_ids == e)
        if len(t_idx) == 0:
            continue
        xe = x[t_idx]
        if quant == QUANT_NONE:
            gu = xe @ bf16_to_f32(w1[e]).T
        elif quant == QUANT_TOKEN_CHANNEL:
            q, s = np_quant(xe, H)
            gu = (tab[q] @ tab[w1[e]].T) * s * w1_scale[e][None, :]
        else:
            q, s = np_quant(xe, 128, quant == QUANT_BLOCK128_UE8M0)
            gu = np.zeros((len(t_idx), I2), np.float32)
            wf = tab[w1[e]]
            for kb in range(H // 128):
                part = tab[q[:, kb * 128:(kb + 1) * 128]] @ wf[:, kb * 128:(kb + 1) * 128].T
                gu += part * s[:, kb:kb + 1] * np.repeat(w1_scale[e][:, kb], 128)[None, :]
        g = gu[:, :I]
        u = np.float32(1) if gate_only else gu[:, I:]
        y = (g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * u
        y = bf16_to_f32(np_f32_to_bf16(y.astype(np.float32)))   # y is held as bf16 in every mode
        if quant == QUANT_NONE:
            o = y @ bf16_to_f32(w2[e]).T
        elif quant == QUANT_TOKEN_CHANNEL:
            q, s = np_quant(y, I)
            o = (tab[q] @ tab[w2[e]].T) * s * w2_scale[e][None, :]
        else:
            q, s = np_quant(y, 128, quant == QUANT_BLOCK128_UE8M0)
            o = np.zeros((len(t_idx), H), np.float32)
            wf = tab[w2[e]]
            for kb in range(I // 128):
                part = tab[q[:, kb * 128:(kb + 1) * 128]] @ wf[:, kb * 128:(kb + 1) * 128].T
                o += part * s[:, kb:kb + 1] * np.repeat(w2_scale[e][:, kb], 128)[None, :]
        part = o.astype(np.float32) * topk_w[t_idx, k_idx][:, None]
        slots[t_idx, k_idx] = bf16_to_f32(np_f32_to_bf16(part)) if partial_bf16 else part
    acc = np.zeros((T, H), np.float32)
    for k in range(K):
        acc += slots[:, k]
    return np_f32_to_bf16(acc)


# ---------------------------------------------------------------------------- configs / inputs

CONFIGS = {
    # name: T, H, I, E, K, quant, routing
    "C0": dict(T=128, H=512, I=1024, E=8, K=2, quant=QUANT_NONE, routing="softmax"),
    "C1": dict(T=4096, H=4096, I=14336, E=8, K=2, quant=QUANT_NONE, routing="softmax"),
    "C2": dict(T=8192, H=4096, I=14336, E=8, K=2, quant=QUANT_TOKEN_CHANNEL, routing="softmax"),
    "C3": dict(T=16, H=4096, I=14336, E=8, K=2, quant=QUANT_TOKEN_CHANNEL, routing="softmax"),
    "C4": dict(T=8192, H=7168, I=2048, E=256, K=8, quant=QUANT_BLOCK128, routing="sigmoid"),
}


def make_inputs(T, H, I, E, K, quant=QUANT_NONE, routing="softmax", seed=0, gate_only=False):
    """Seeded synthetic inputs: activations N(0,1), weights N(0,0.02), logits N(0,1)."""
    x = f32_to_bf16(normal((T, H), seed, 1))
    R1 = I if gate_only else 2 * I
    w1f = normal((E, R1, H), seed, 2, 0.02)
    w2f = normal((E, H, I), seed, 3, 0.02)
    logits = normal((T, E), seed, 4)
    ids, w = route(logits, K, routing)
    d = dict(x=x, topk_ids=ids, topk_w=w, logits=logits, quant=quant, w1_scale=None, w2_scale=None)
    if quant == QUANT_NONE:
        d["w1"], d["w2"] = f32_to_bf16(w1f), f32_to_bf16(w2f)
    elif quant == QUANT_TOKEN_CHANNEL:
        q1, s1 = quant_rows_e4m3(w1f.reshape(E * R1, H))
        q2, s2 = quant_rows_e4m3(w2f.reshape(E * H, I))
        d["w1"], d["w1_scale"] = q1.reshape(E, R1, H), s1.reshape(E, R1)
        d["w2"], d["w2_scale"] = q2.reshape(E, H, I), s2.reshape(E, H)
    else:
        pow2 = quant == QUANT_BLOCK128_UE8M0
        q1, s1 = quant_blocks_e4m3(w1f.reshape(E * R1, H), pow2)
        q2, s2 = quant_blocks_e4m3(w2f.reshape(E * H, I), pow2)
        d["w1"], d["w1_scale"] = q1.reshape(E, R1, H), s1.reshape(E, R1 // 128, H // 128)
        d["w2"], d["w2_scale"] = q2.reshape(E, H, I), s2.reshape(E, H // 128, I // 128)
    return d
