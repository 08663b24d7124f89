"""numpy front-end to the C oracle (``ab_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA library and the timed CPU
baseline.  Nothing in the shipped package imports this module.  Each wrapper
names the oracle function it calls; the C source cites the reference file:line
each function restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_SRC = os.path.join(_HERE, "ab_oracle.c")


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    stale = (not os.path.exists(_SO)) or (
        os.path.exists(_SRC) and os.path.getmtime(_SRC) > os.path.getmtime(_SO))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-s"] + (["-B"] if force else []), check=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def _declare(L):
    L.orc_num_threads.restype = C.c_int
    L.orc_set_threads.argtypes = [C.c_int]; L.orc_set_threads.restype = None
    L.orc_f32_to_f16.argtypes = [C.c_float]; L.orc_f32_to_f16.restype = C.c_uint16
    L.orc_f32_to_f16_rne.argtypes = [C.c_float]; L.orc_f32_to_f16_rne.restype = C.c_uint16
    L.orc_f16_to_f32.argtypes = [C.c_uint16]; L.orc_f16_to_f32.restype = C.c_float
    L.orc_bf16_to_f32.argtypes = [C.c_uint16]; L.orc_bf16_to_f32.restype = C.c_float
    L.orc_f32_to_bf16.argtypes = [C.c_float]; L.orc_f32_to_bf16.restype = C.c_uint16
    L.orc_quantise_absmax_i8.argtypes = [_f32p, C.c_size_t, _i8p]
    L.orc_quantise_absmax_i8.restype = C.c_float
    L.orc_dequantise_i8.argtypes = [_i8p, C.c_size_t, C.c_float, _f32p]
    L.orc_quantise_absmax_i8_rows.argtypes = [_f32p, C.c_int, C.c_int, _i8p, _f32p]
    L.orc_dequantise_i8_rows.argtypes = [_i8p, C.c_int, C.c_int, _f32p, _f32p]
    L.orc_pack_i4.argtypes = [_u8p, C.c_size_t, _u8p]
    L.orc_unpack_i4.argtypes = [_u8p, C.c_size_t, _u8p]
    L.orc_quantise_affine_i4.argtypes = [_f32p, C.c_size_t, C.c_size_t, _u8p, _f32p, _f32p]
    L.orc_dequantise_i4.argtypes = [_u8p, C.c_size_t, C.c_size_t, _f32p, _f32p, _f32p]
    L.orc_quantise_block_q4km.argtypes = [_f32p, _u8p]
    L.orc_dequantise_block_q4km.argtypes = [_u8p, _f32p]
    L.orc_encode_q4km_tensor.argtypes = [_f32p, C.c_size_t, _u8p]
    L.orc_decode_q4km_tensor.argtypes = [_u8p, C.c_size_t, _f32p]
    L.orc_fake_quant_export_q4km.argtypes = [_f32p, C.c_size_t, _f32p]
    L.orc_dequant_w4a16.argtypes = [_u32p, _u16p, _u32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
    L.orc_linear_f32.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
    L.orc_linear_f64acc.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
    L.orc_rms_norm_scalar.argtypes = [_f32p, _f32p, C.c_float, _f32p, C.c_int, C.c_int]
    L.orc_rms_norm_avx2fma_order.argtypes = [_f32p, _f32p, C.c_float, _f32p, C.c_int, C.c_int]
    L.orc_rope_tables.argtypes = [C.c_int, C.c_int, C.c_double, _f32p, _f32p]
    L.orc_rope_apply.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int] * 5
    L.orc_swiglu.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
    L.orc_attention.argtypes = [_f32p, _f32p, _f32p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                C.c_float, _f32p] + [C.c_int] * 6
    L.orc_attention_decode_gqa.argtypes = [_f32p, _f32p, _f32p, _i32p, C.c_int, C.c_float, _f32p,
                                           C.c_int, C.c_int, C.c_int, C.c_int]
    L.orc_quantise_kv_rows.argtypes = [_f32p, C.c_long, C.c_int, _i8p, _f32p]
    L.orc_argmax.argtypes = [_f32p, C.c_int]; L.orc_argmax.restype = C.c_int
    L.orc_model_create.argtypes = [C.c_int] * 8 + [C.c_float, C.c_double, C.c_int, C.c_int]
    L.orc_model_create.restype = C.c_void_p
    L.orc_model_set_weight.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p]
    L.orc_model_set_norm_order.argtypes = [C.c_void_p, C.c_int]
    L.orc_model_set_linear_order.argtypes = [C.c_void_p, C.c_int]
    L.orc_model_reset.argtypes = [C.c_void_p]
    L.orc_model_seq_len.argtypes = [C.c_void_p, C.c_int]; L.orc_model_seq_len.restype = C.c_int
    L.orc_model_truncate.argtypes = [C.c_void_p, C.c_int, C.c_int]
    L.orc_model_truncate.restype = C.c_int
    L.orc_model_destroy.argtypes = [C.c_void_p]
    L.orc_model_fill_cache.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint32]
    L.orc_model_forward.argtypes = [C.c_void_p, _u32p, C.c_int, C.c_int, C.c_int, _i32p, _f32p]
    L.orc_model_forward.restype = C.c_int


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads() -> int:
    return lib().orc_num_threads()


def use_all_cores() -> int:
    """Runs the parallel loops on every core this process may use (a launcher
    such as torchrun exports OMP_NUM_THREADS=1 to its workers); returns the count."""
    import os
    n = len(os.sched_getaffinity(0))
    lib().orc_set_threads(n)
    return num_threads()


# --- f16 / bf16 -------------------------------------------------------------
def f32_to_f16(v: float) -> int:
    return int(lib().orc_f32_to_f16(float(np.float32(v))))


def f32_to_f16_rne(v: float) -> int:
    return int(lib().orc_f32_to_f16_rne(float(np.float32(v))))


def f16_to_f32(bits: int) -> np.float32:
    return np.float32(lib().orc_f16_to_f32(int(bits)))


def bf16_bits(a) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    x = _f32(a).view(np.uint32).astype(np.uint64)
    lsb = (x >> 16) & 1
    return (((x + 0x7FFF + lsb) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(a) -> np.ndarray:
    return bf16_to_f32(bf16_bits(a))


# --- INT8 -------------------------------------------------------------------
def quantise_absmax_i8(values):
    v = _f32(values).ravel()
    codes = np.empty(v.size, np.int8)
    scale = lib().orc_quantise_absmax_i8(v, v.size, codes)
    return codes.reshape(np.shape(values)), np.float32(scale)


def dequantise_i8(codes, scale):
    c = np.ascontiguousarray(codes, np.int8)
    out = np.empty(c.size, np.float32)
    lib().orc_dequantise_i8(c.ravel(), c.size, float(scale), out)
    return out.reshape(c.shape)


def quantise_absmax_i8_rows(w):
    w = _f32(w)
    N, K = w.shape
    codes = np.empty((N, K), np.int8)
    scales = np.empty(N, np.float32)
    lib().orc_quantise_absmax_i8_rows(w, N, K, codes, scales)
    return codes, scales


def dequantise_i8_rows(codes, scales):
    c = np.ascontiguousarray(codes, np.int8)
    N, K = c.shape
    out = np.empty((N, K), np.float32)
    lib().orc_dequantise_i8_rows(c, N, K, _f32(scales), out)
    return out


# --- INT4 affine ------------------------------------------------------------
def pack_i4(values):
    v = np.ascontiguousarray(values, np.uint8).ravel()
    packed = np.zeros((v.size + 1) // 2, np.uint8)
    lib().orc_pack_i4(v, v.size, packed)
    return packed


def unpack_i4(packed, n):
    p = np.ascontiguousarray(packed, np.uint8).ravel()
    out = np.empty(n, np.uint8)
    lib().orc_unpack_i4(p, n, out)
    return out


def quantise_affine_i4(values, group):
    v = _f32(values).ravel()
    ng = (v.size + group - 1) // group
    packed = np.zeros((v.size + 1) // 2, np.uint8)
    scales = np.empty(ng, np.float32)
    zeros = np.empty(ng, np.float32)
    lib().orc_quantise_affine_i4(v, v.size, group, packed, scales, zeros)
    return packed, scales, zeros


def dequantise_i4(packed, n, group, scales, zeros):
    out = np.empty(n, np.float32)
    lib().orc_dequantise_i4(np.ascontiguousarray(packed, np.uint8), n, group, _f32(scales),
                            _f32(zeros), out)
    return out


# --- Q4_K_M-style blocks ----------------------------------------------------
def quantise_block_q4km(w256):
    enc = np.empty(132, np.uint8)
    lib().orc_quantise_block_q4km(_f32(w256), enc)
    return enc


def dequantise_block_q4km(enc):
    out = np.empty(256, np.float32)
    lib().orc_dequantise_block_q4km(np.ascontiguousarray(enc, np.uint8), out)
    return out


def encode_q4km_tensor(values):
    v = _f32(values).ravel()
    payload = np.empty(((v.size + 255) // 256) * 132, np.uint8)
    lib().orc_encode_q4km_tensor(v, v.size, payload)
    return payload


def decode_q4km_tensor(payload, shape):
    n = int(np.prod(shape))
    out = np.empty(n, np.float32)
    lib().orc_decode_q4km_tensor(np.ascontiguousarray(payload, np.uint8), n, out)
    return out.reshape(shape)


def fake_quant_export_q4km(values):
    v = _f32(values).ravel()
    out = np.empty(v.size, np.float32)
    lib().orc_fake_quant_export_q4km(v, v.size, out)
    return out.reshape(np.shape(values))


# --- W4A16 ------------------------------------------------------------------
def dequant_w4a16(qweight, scales_bf16, qzeros, N, K, group, awq_order=False):
    out = np.empty((N, K), np.float32)
    lib().orc_dequant_w4a16(np.ascontiguousarray(qweight, np.uint32),
                            np.ascontiguousarray(scales_bf16, np.uint16),
                            np.ascontiguousarray(qzeros, np.uint32), N, K, group,
                            1 if awq_order else 0, out)
    return out


# --- ops --------------------------------------------------------------------
def linear(x, w, f64acc=False):
    x = _f32(x); w = _f32(w)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), np.float32)
    (lib().orc_linear_f64acc if f64acc else lib().orc_linear_f32)(x, w, y, M, N, K)
    return y


def rms_norm(x, w, eps, simd_order=True):
    x = _f32(x)
    d = x.shape[-1]
    rows = x.size // d
    out = np.empty_like(x)
    fn = lib().orc_rms_norm_avx2fma_order if simd_order else lib().orc_rms_norm_scalar
    fn(x.reshape(rows, d), _f32(w), eps, out.reshape(rows, d), rows, d)
    return out


def rope_tables(max_seq, head_dim, theta=10000.0):
    cos = np.empty((max_seq, head_dim // 2), np.float32)
    sin = np.empty((max_seq, head_dim // 2), np.float32)
    lib().orc_rope_tables(max_seq, head_dim, theta, cos, sin)
    return cos, sin


def rope_apply(x, cos, sin, offset):
    x = _f32(x)
    b, s, h, hd = x.shape
    out = np.empty_like(x)
    lib().orc_rope_apply(x, out, _f32(cos), _f32(sin), b, s, h, hd, offset)
    return out


def swiglu(gate, up):
    g = _f32(gate); u = _f32(up)
    out = np.empty_like(g)
    lib().orc_swiglu(g.ravel(), u.ravel(), out.ravel(), g.size)
    return out


def attention(q, k, v, scale, mask=None, causal=False, parallel=True):
    q = _f32(q); k = _f32(k); v = _f32(v)
    b, h, qs, hd = q.shape
    kvs = k.shape[2]
    out = np.empty_like(q)
    if mask is not None:
        mask = _f32(mask)
        mp, mb, mh = mask.ctypes.data_as(C.c_void_p), mask.shape[0], mask.shape[1]
    else:
        mp, mb, mh = None, 1, 1
    lib().orc_attention(q, k, v, mp, mb, mh, 1 if causal else 0, scale, out, b, h, qs, kvs, hd,
                        1 if parallel else 0)
    return out


def attention_decode_gqa(q, kc, vc, kv_lens, scale):
    """q [b,h,hd]; kc,vc [b,cap,kvh,hd]; kv_lens [b]."""
    q = _f32(q); kc = _f32(kc); vc = _f32(vc)
    b, h, hd = q.shape
    cap, kvh = kc.shape[1], kc.shape[2]
    out = np.empty_like(q)
    lib().orc_attention_decode_gqa(q, kc, vc, np.ascontiguousarray(kv_lens, np.int32), cap, scale,
                                   out, b, h, kvh, hd)
    return out


def quantise_kv_rows(x):
    """Per-(token, head) symmetric INT8 over the last axis."""
    x = _f32(x)
    hd = x.shape[-1]
    rows = x.size // hd
    codes = np.empty(x.shape, np.int8)
    scales = np.empty(x.shape[:-1], np.float32)
    lib().orc_quantise_kv_rows(x.reshape(rows, hd), rows, hd, codes.reshape(rows, hd),
                               scales.reshape(rows))
    return codes, scales


def argmax(values) -> int:
    v = _f32(values).ravel()
    return int(lib().orc_argmax(v, v.size))


# --- reference KV-cache semantics (host-only structures) --------------------
class KVCache:
    """KVCache with preallocated storage (crates/aarambh-studio-nn/src/kvcache.rs:236-369)."""

    def __init__(self, capacity=None):
        self.k = None
        self.v = None
        self.len = 0
        self.capacity = capacity

    def update(self, k, v):
        k = _f32(k); v = _f32(v)
        if self.capacity is None:
            self.k = k if self.k is None else np.concatenate([self.k[:, :self.len], k], 1)
            self.v = v if self.v is None else np.concatenate([self.v[:, :self.len], v], 1)
            self.len = self.k.shape[1]
            return self.k, self.v
        if k.ndim != 4 or v.shape != k.shape:
            raise ValueError("KV cache expects matching rank-4 tensors")
        s = k.shape[1]
        if self.len + s > self.capacity:
            raise ValueError(f"KV cache length {self.len + s} exceeds capacity {self.capacity}")
        if self.k is None:
            shape = (k.shape[0], self.capacity, k.shape[2], k.shape[3])
            self.k = np.zeros(shape, np.float32)
            self.v = np.zeros(shape, np.float32)
        self.k[:, self.len:self.len + s] = k
        self.v[:, self.len:self.len + s] = v
        self.len += s
        return self.k[:, :self.len], self.v[:, :self.len]

    def truncate(self, new_len):
        if new_len > self.len:
            raise ValueError(f"cannot grow KV cache from {self.len} to {new_len} with truncate")
        self.len = new_len
        if self.capacity is None and new_len == 0:
            self.k = self.v = None

    def clear(self):
        self.len = 0
        if self.capacity is None:
            self.k = self.v = None

    def seq_len(self):
        return self.len


class QuantisedKvCache:
    """Per-tensor INT8 cache that re-quantises everything on each append
    (crates/aarambh-studio-quant/src/kv_quant.rs:16-74)."""

    def __init__(self, n_layers):
        self.layers = [dict(k=None, v=None) for _ in range(n_layers)]

    def append_and_get(self, layer, k, v):
        c = self.layers[layer]
        k = _f32(k); v = _f32(v)
        k_full = k if c["k"] is None else np.concatenate([dequantise_i8(*c["k"]), k], 1)
        v_full = v if c["v"] is None else np.concatenate([dequantise_i8(*c["v"]), v], 1)
        c["k"] = quantise_absmax_i8(k_full)
        c["v"] = quantise_absmax_i8(v_full)
        return k_full, v_full

    def seq_len(self, layer):
        c = self.layers[layer]["k"]
        return 0 if c is None else c[0].shape[1]

    def clear(self):
        for c in self.layers:
            c["k"] = c["v"] = None


# --- dense decoder (the reference's CPU inference path) ----------------------
class DenseModel:
    """Dense f32 decoder with per-sequence KV caches; see ``orc_model_forward``."""

    PER_LAYER = ["wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down", "norm1", "norm2"]

    def __init__(self, cfg: dict, weights: dict, batch: int, capacity: int):
        self.cfg = cfg
        self._keep = []
        L = lib()
        self.h = L.orc_model_create(cfg["n_layers"], cfg["d_model"], cfg["n_heads"],
                                    cfg["n_kv_heads"], cfg["head_dim"], cfg["ffn_hidden"],
                                    cfg["vocab"], cfg["max_seq"], cfg.get("eps", 1e-5),
                                    cfg.get("rope_theta", 10000.0), batch, capacity)
        for name, which in (("embedding", 0), ("lm_head", 1), ("final_norm", 2)):
            a = _f32(weights[name]); self._keep.append(a)
            L.orc_model_set_weight(self.h, -1, which, a.reshape(-1))
        for l in range(cfg["n_layers"]):
            for which, name in enumerate(self.PER_LAYER):
                a = _f32(weights[f"layers.{l}.{name}"]); self._keep.append(a)
                L.orc_model_set_weight(self.h, l, which, a.reshape(-1))

    def forward(self, ids, offsets, row0=0):
        ids = np.ascontiguousarray(ids, np.uint32)
        B, S = ids.shape
        logits = np.empty((B, S, self.cfg["vocab"]), np.float32)
        rc = lib().orc_model_forward(self.h, ids, B, S, row0,
                                     np.ascontiguousarray(offsets, np.int32), logits)
        if rc != 0:
            raise ValueError("KV cache capacity or max_seq_len exceeded")
        return logits

    def set_linear_order(self, lanes: bool):
        """False: strict k order per output (the parity definition); True: 16-lane SIMD
        order with FMA, for the timed CPU baseline only."""
        lib().orc_model_set_linear_order(self.h, 1 if lanes else 0)

    def fill_cache(self, row, length, seed=1):
        lib().orc_model_fill_cache(self.h, row, length, seed)

    def reset(self):
        lib().orc_model_reset(self.h)

    def seq_len(self, b=0):
        return lib().orc_model_seq_len(self.h, b)

    def truncate(self, b, new_len):
        if lib().orc_model_truncate(self.h, b, new_len) != 0:
            raise ValueError("cannot grow KV cache with truncate")

    def __del__(self):
        try:
            lib().orc_model_destroy(self.h)
        except Exception:
            pass
