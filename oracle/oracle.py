"""ctypes front-end of the CPU oracle.  TEST INFRASTRUCTURE — never imported by the product package.

Only tests/, the smoke check and the CPU-baseline / reference arm of bench.py
may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libnerva_oracle.so")

MODE_CPU = 0
MODE_CUDA = 1
DTYPE_F16 = 0
DTYPE_BF16 = 1

_u16p = C.POINTER(C.c_uint16)
_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)


class OracleLayer(C.Structure):
    _fields_ = [(n, _u16p) for n in (
        "rms_attn", "rms_mlp", "w_q", "w_k", "w_v", "w_o", "q_norm", "k_norm",
        "q_bias", "k_bias", "v_bias", "o_bias", "w_gate", "w_up", "w_down")] + [
        (n, C.c_uint32) for n in (
            "mlp_kind", "moe_intermediate", "shared_intermediate", "num_experts", "top_k", "norm_topk_prob")] + [
        (n, _u16p) for n in (
            "w_router", "w_expert_gate_up", "w_expert_down",
            "w_shared_gate", "w_shared_up", "w_shared_down", "w_shared_router")] + [
        (n, C.c_uint32) for n in ("attention_kind", "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim")] + [
        (n, _u16p) for n in ("w_kv_a", "kv_a_norm", "w_kv_b")]


class OracleModel(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "dtype", "hidden", "heads", "kv_heads", "head_dim", "intermediate", "vocab", "layers")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_float),
        ("embeddings", _u16p), ("final_norm", _u16p), ("lm_head", _u16p),
        ("layer", C.POINTER(OracleLayer))]


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file."""
    # make decides what is stale (a source newer than the library)
    if force:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    else:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.oracle_bf16_to_f32.restype = C.c_float
        L.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_bf16.restype = C.c_uint16
        L.oracle_f32_to_bf16.argtypes = [C.c_float]
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_silu.restype = C.c_float
        L.oracle_silu.argtypes = [C.c_float]
        L.oracle_rms_norm.argtypes = [C.c_uint32, _f32p, _u16p, C.c_uint32, C.c_float, _f32p]
        L.oracle_per_head_rms_norm.argtypes = [C.c_uint32, _u16p, C.c_uint32, _f32p, C.c_uint32, C.c_float]
        L.oracle_matvec.argtypes = [C.c_uint32, _u16p, _f32p, C.c_uint32, C.c_uint32, _f32p]
        L.oracle_rope.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float]
        L.oracle_attention.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _f32p]
        L.oracle_attention_paged.argtypes = [C.c_uint32, _f32p, _u16p, _u16p, _u32p, C.c_uint32, C.c_uint32,
                                             C.c_uint32, C.c_uint32, _f32p]
        L.oracle_argmax.restype = C.c_int64
        L.oracle_argmax.argtypes = [_f32p, C.c_uint32, C.c_int]
        L.oracle_route_softmax_topk.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_uint32, _u32p, _f32p]
        L.oracle_create.restype = C.c_void_p
        L.oracle_create.argtypes = [C.POINTER(OracleModel), C.c_uint32, C.c_int]
        L.oracle_destroy.argtypes = [C.c_void_p]
        L.oracle_reset.argtypes = [C.c_void_p]
        L.oracle_position.restype = C.c_uint32
        L.oracle_position.argtypes = [C.c_void_p]
        L.oracle_step.argtypes = [C.c_void_p, C.c_uint32, _f32p]
        L.oracle_decode_greedy.argtypes = [C.c_void_p, _u32p, C.c_uint32, C.c_uint32, _u32p, _f32p]
        L.oracle_hidden_state.restype = _f32p
        L.oracle_hidden_state.argtypes = [C.c_void_p]
        L.oracle_hash_tokens.restype = C.c_uint64
        L.oracle_hash_tokens.argtypes = [_u32p, C.c_uint32]
        L.oracle_set_threads.argtypes = [C.c_int]
        L.oracle_set_sum_lanes.argtypes = [C.c_int]
        L.oracle_get_threads.restype = C.c_int
        _lib = L
    return _lib


def _p16(a):
    return None if a is None else a.ctypes.data_as(_u16p)


def synth_normal_bf16(seed: int, tensor_id: int, count: int, std: float) -> np.ndarray:
    """Multi-threaded twin of nerva_b200.synth.normal_bf16 (same bits), inside the oracle library."""
    out = np.empty(count, dtype=np.uint16)
    fn = lib().oracle_synth_normal_bf16
    fn.restype = None
    fn.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, _u16p]
    fn(seed, tensor_id, count, std, _p16(out))
    return out


def synth_normal_bf16_block(seed: int, tensor_id: int, full_cols: int, row_begin: int, rows: int, col_begin: int,
                            cols: int, std: float) -> np.ndarray:
    """A rows x cols block of the row-major synthetic tensor with `full_cols` columns, flattened."""
    out = np.empty(rows * cols, dtype=np.uint16)
    fn = lib().oracle_synth_normal_bf16_block
    fn.restype = None
    fn.argtypes = [C.c_uint64] * 7 + [C.c_float, _u16p]
    fn(seed, tensor_id, full_cols, row_begin, rows, col_begin, cols, std, _p16(out))
    return out


def _pf(a):
    return a.ctypes.data_as(_f32p)


def _pu(a):
    return a.ctypes.data_as(_u32p)


def matvec(matrix_bits: np.ndarray, x: np.ndarray, rows: int, cols: int, dtype: int = DTYPE_BF16) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(rows, dtype=np.float32)
    lib().oracle_matvec(dtype, _p16(matrix_bits), _pf(x), rows, cols, _pf(out))
    return out


def rms_norm(x: np.ndarray, weight_bits: np.ndarray, eps: float, dtype: int = DTYPE_BF16) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().oracle_rms_norm(dtype, _pf(x), _p16(weight_bits), x.size, eps, _pf(out))
    return out


def per_head_rms_norm(values: np.ndarray, weight_bits: np.ndarray, head_dim: int, eps: float,
                      dtype: int = DTYPE_BF16) -> np.ndarray:
    out = np.array(values, dtype=np.float32, copy=True)
    lib().oracle_per_head_rms_norm(dtype, _p16(weight_bits), head_dim, _pf(out), out.size, eps)
    return out


def rope(values: np.ndarray, heads: int, head_dim: int, position: int, theta: float) -> np.ndarray:
    out = np.array(values, dtype=np.float32, copy=True)
    lib().oracle_rope(_pf(out), heads, head_dim, position, theta)
    return out


def attention(q, keys, values, tokens, heads, kv_heads, head_dim) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    keys = np.ascontiguousarray(keys, dtype=np.float32)
    values = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(heads * head_dim, dtype=np.float32)
    rc = lib().oracle_attention(_pf(q), _pf(keys), _pf(values), tokens, heads, kv_heads, head_dim, _pf(out))
    if rc != 0:
        raise ValueError("oracle attention rejected its input")
    return out


def attention_paged(q, key_pages, value_pages, page_table, tokens, heads, kv_heads, head_dim,
                    dtype: int = DTYPE_BF16) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    page_table = np.ascontiguousarray(page_table, dtype=np.uint32)
    out = np.empty(heads * head_dim, dtype=np.float32)
    rc = lib().oracle_attention_paged(dtype, _pf(q), _p16(key_pages), _p16(value_pages), _pu(page_table),
                                      tokens, heads, kv_heads, head_dim, _pf(out))
    if rc != 0:
        raise ValueError("oracle paged attention rejected its input")
    return out


def argmax(logits: np.ndarray, mode: int = MODE_CUDA) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().oracle_argmax(_pf(logits), logits.size, mode))


def route_softmax_topk(router_logits, top_k: int, norm_topk_prob: bool):
    logits = np.ascontiguousarray(router_logits, dtype=np.float32)
    experts = np.zeros(top_k, dtype=np.uint32)
    weights = np.zeros(top_k, dtype=np.float32)
    lib().oracle_route_softmax_topk(_pf(logits), logits.size, top_k, int(norm_topk_prob), _pu(experts), _pf(weights))
    return experts, weights


def set_sum_lanes(lanes: int) -> None:
    """1 = reference serial summation; n > 1 = a different, equally valid fp32 order."""
    lib().oracle_set_sum_lanes(lanes)


def hash_tokens(tokens) -> int:
    t = np.ascontiguousarray(tokens, dtype=np.uint32)
    return int(lib().oracle_hash_tokens(_pu(t), t.size))


class Decoder:
    """CPU decoder over a checkpoint object exposing `.config`, `.embeddings`,
    `.final_norm`, `.lm_head` and `.layers` (list of dict name -> uint16 array)."""

    def __init__(self, checkpoint, max_context: int, mode: int = MODE_CPU, dtype: int = DTYPE_BF16):
        cfg = checkpoint.config
        self.cfg = cfg
        self._keep = checkpoint
        self._layers = (OracleLayer * cfg.layers)()
        names = {"w_shared_gate": "w_shared_expert_gate", "w_shared_up": "w_shared_expert_up",
                 "w_shared_down": "w_shared_expert_down", "w_shared_router": "w_shared_expert_router"}
        for i, entry in enumerate(checkpoint.layers):
            layer = self._layers[i]
            for fname, ftype in OracleLayer._fields_:
                if ftype is _u16p:
                    setattr(layer, fname, _p16(entry.get(names.get(fname, fname))))
            if getattr(cfg, "kv_lora_rank", 0):
                layer.attention_kind = 2
                layer.kv_lora_rank = cfg.kv_lora_rank
                layer.qk_nope_head_dim = cfg.qk_nope_head_dim
                layer.qk_rope_head_dim = cfg.qk_rope_head_dim
            if cfg.num_experts and i >= getattr(cfg, "dense_layers", 0):
                layer.mlp_kind = 1
                layer.moe_intermediate = cfg.moe_intermediate
                layer.shared_intermediate = cfg.shared_intermediate
                layer.num_experts = cfg.num_experts
                layer.top_k = cfg.top_k
                layer.norm_topk_prob = int(cfg.norm_topk_prob)
        self._model = OracleModel(
            dtype=dtype, hidden=cfg.hidden, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
            intermediate=cfg.intermediate, vocab=cfg.vocab, layers=cfg.layers, rms_eps=cfg.rms_eps,
            rope_theta=cfg.rope_theta, embeddings=_p16(checkpoint.embeddings),
            final_norm=_p16(checkpoint.final_norm), lm_head=_p16(checkpoint.lm_head),
            layer=C.cast(self._layers, C.POINTER(OracleLayer)))
        self._ctx = lib().oracle_create(C.byref(self._model), max_context, mode)
        if not self._ctx:
            raise ValueError("oracle rejected the model")
        self.mode = mode

    def close(self):
        if self._ctx:
            lib().oracle_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        self.close()

    def reset(self):
        lib().oracle_reset(self._ctx)

    def seek_for_timing(self, position: int) -> None:
        """Jump to `position` with a patterned cache: later steps cost what they cost after a real
        prefill of that length, their tokens mean nothing (bounded CPU timing samples only)."""
        fn = lib().oracle_seek_for_timing
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_uint32]
        if fn(self._ctx, position) != 0:
            raise ValueError("seek rejected")

    def step(self, token: int, want_logits: bool = True):
        logits = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        rc = lib().oracle_step(self._ctx, int(token), _pf(logits) if want_logits else None)
        if rc != 0:
            raise ValueError("oracle step failed")
        return logits

    def hidden_state(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().oracle_hidden_state(self._ctx), shape=(self.cfg.hidden,)).copy()

    def decode_greedy(self, prompt, steps: int, want_logits: bool = False):
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        tokens = np.zeros(steps, dtype=np.uint32)
        logits = np.empty((steps, self.cfg.vocab), dtype=np.float32) if want_logits else None
        n = lib().oracle_decode_greedy(self._ctx, _pu(prompt), prompt.size, steps, _pu(tokens),
                                       _pf(logits) if want_logits else None)
        if n < 0:
            raise ValueError("oracle decode failed")
        return (tokens[:n], logits[:n]) if want_logits else tokens[:n]


# ---- DeepSeek expert routers (oracle/nerva_oracle_router.c) and the reference's own header ----

_REF_ROUTER_PATH = os.path.join(_HERE, "_ref", "libnerva_ref_router.so")
# the reference checkout: NERVA_REFERENCE_ROOT, else a directory `reference` beside this repository
REFERENCE_ROOT = os.environ.get("NERVA_REFERENCE_ROOT",
                                 os.path.abspath(os.path.join(_HERE, "..", "..", "reference")))
_REFERENCE_HEADER = os.path.join(REFERENCE_ROOT, "native/cuda/deepseek/deepseek_router.cuh")
_REF_SAMPLER_PATH = os.path.join(_HERE, "_ref", "libnerva_ref_sampler.so")
_ref_router = None
_ref_sampler = None


def build_ref(force: bool = False):
    """Compiles the reference's router header for the host (oracle/_ref/), where the reference
    checkout exists.  Returns the library path, or None when neither checkout nor a prebuilt
    library is there."""
    if os.path.exists(_REFERENCE_HEADER) and (force or not os.path.exists(_REF_ROUTER_PATH)
                                              or not os.path.exists(_REF_SAMPLER_PATH)):
        subprocess.run(["make", "-C", _HERE, "ref", f"REFERENCE_ROOT={REFERENCE_ROOT}"], check=True, capture_output=True)
    return _REF_ROUTER_PATH if os.path.exists(_REF_ROUTER_PATH) else None


def ref_router_lib():
    """The reference router compiled for the host, or None when it has not been built."""
    global _ref_router
    if _ref_router is None:
        path = build_ref()
        if path is None:
            return None
        _ref_router = C.CDLL(path)
    return _ref_router


def _route(fn, kind: str, logits, bias, top_k, norm_topk_prob, scaling, num_groups=0, top_k_groups=0, table=None,
           route_token=0):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    bias_arr = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    ids = np.zeros(top_k, dtype=np.uint32)
    weights = np.zeros(top_k, dtype=np.float32)
    f = C.c_float(scaling)
    if kind == "v3":
        rc = fn(_pf(logits), _pf(bias_arr) if bias_arr is not None else None, logits.size, num_groups, top_k_groups,
                top_k, int(norm_topk_prob), f, _pu(ids), _pf(weights))
    elif kind == "v4":
        rc = fn(_pf(logits), _pf(bias_arr) if bias_arr is not None else None, logits.size, top_k,
                int(norm_topk_prob), f, _pu(ids), _pf(weights))
    else:
        table = np.ascontiguousarray(table, dtype=np.uint32)
        rc = fn(_pf(logits), _pu(table), table.size, route_token, logits.size, top_k, int(norm_topk_prob), f,
                _pu(ids), _pf(weights))
    return rc, ids, weights


def _router_fn(library, prefix: str, kind: str):
    name = {"v3": "route_v3_grouped_sigmoid", "v4": "route_v4_sqrtsoftplus", "hash": "route_v4_hash"}[kind]
    fn = getattr(library, f"{prefix}_{name}")
    fn.restype = C.c_int
    fn.argtypes = None  # mixed pointer / scalar arguments are passed explicitly typed by _route
    return fn


def route_v3_grouped_sigmoid(logits, bias, num_groups, top_k_groups, top_k, norm_topk_prob, scaling, ref=False):
    library = ref_router_lib() if ref else lib()
    return _route(_router_fn(library, "ref" if ref else "oracle", "v3"), "v3", logits, bias, top_k, norm_topk_prob,
                  scaling, num_groups=num_groups, top_k_groups=top_k_groups)


def route_v4_sqrtsoftplus(logits, bias, top_k, norm_topk_prob, scaling, ref=False):
    library = ref_router_lib() if ref else lib()
    return _route(_router_fn(library, "ref" if ref else "oracle", "v4"), "v4", logits, bias, top_k, norm_topk_prob,
                  scaling)


def route_v4_hash(logits, table, route_token, top_k, norm_topk_prob, scaling, ref=False):
    library = ref_router_lib() if ref else lib()
    return _route(_router_fn(library, "ref" if ref else "oracle", "hash"), "hash", logits, None, top_k,
                  norm_topk_prob, scaling, table=table, route_token=route_token)


# ---- DeepSeek MLA decode (oracle/nerva_oracle_mla.c) ----

def mla_decode(q_nope, q_pe, kv_c, k_pe, w_uk, w_uv, heads, tokens, kv_lora_rank, qk_nope_head_dim,
               qk_rope_head_dim, v_head_dim, softmax_scale):
    """Absorbed multi-head latent attention for one token; returns (status, out [heads * v_head_dim])."""
    arrays = [np.ascontiguousarray(a, dtype=np.float32) for a in (q_nope, q_pe, kv_c, k_pe, w_uk, w_uv)]
    out = np.zeros(heads * v_head_dim, dtype=np.float32)
    fn = lib().oracle_mla_decode
    fn.restype = C.c_int
    fn.argtypes = [_f32p] * 7 + [C.c_uint32] * 6 + [C.c_float]
    rc = fn(*[_pf(a) for a in arrays], _pf(out), heads, tokens, kv_lora_rank, qk_nope_head_dim, qk_rope_head_dim,
            v_head_dim, softmax_scale)
    return rc, out


def moe_forward(x, expert_ids, expert_weights, w_gate, w_up, w_down, hidden, intermediate, num_experts,
                clamp_swiglu=False, swiglu_limit=0.0):
    """fp32 expert MLP of one token; returns (status, out [hidden])."""
    x, w_gate, w_up, w_down, ew = [np.ascontiguousarray(a, dtype=np.float32)
                                   for a in (x, w_gate, w_up, w_down, expert_weights)]
    ids = np.ascontiguousarray(expert_ids, dtype=np.uint32)
    out = np.zeros(hidden, dtype=np.float32)
    fn = lib().oracle_moe_forward
    fn.restype = C.c_int
    fn.argtypes = [_f32p, _u32p, _f32p, _f32p, _f32p, _f32p, _f32p] + [C.c_uint32] * 5 + [C.c_float]
    rc = fn(_pf(x), _pu(ids), _pf(ew), _pf(w_gate), _pf(w_up), _pf(w_down), _pf(out), hidden, intermediate,
            num_experts, ids.size, int(clamp_swiglu), swiglu_limit)
    return rc, out


def sampler_uniform(seed: int, position: int, token: int, salt: int) -> float:
    fn = lib().oracle_sampler_uniform
    fn.restype = C.c_float
    fn.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]
    return fn(seed, position, token, salt)


def sample_token(logits, position: int, temperature: float, top_p: float, top_k: int, seed: int):
    """Restated sampler: returns (token, margin), margin being the relative distance of the
    closest comparison the choice depended on (inf for arg-max)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    fn = lib().oracle_sample_token
    fn.restype = C.c_uint32
    fn.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_uint32, C.c_uint64, _f32p]
    margin = C.c_float(0.0)
    token = fn(_pf(logits), logits.size, position, temperature, top_p, top_k, seed, C.byref(margin))
    return token, margin.value


def ref_sampler_lib():
    """The reference's sampler kernel behind a host wrapper (needs a GPU to run), or None."""
    global _ref_sampler
    if _ref_sampler is None:
        build_ref()
        if not os.path.exists(_REF_SAMPLER_PATH):
            return None
        _ref_sampler = C.CDLL(_REF_SAMPLER_PATH)
        _ref_sampler.ref_sample_token.restype = C.c_int
        _ref_sampler.ref_sample_token.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_uint32,
                                                  C.c_uint64, _u32p]
    return _ref_sampler


def ref_sample_token(logits, position: int, temperature: float, top_p: float, top_k: int, seed: int) -> int:
    """One token from the reference's own kernel on the current CUDA device."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    token = C.c_uint32(0)
    rc = ref_sampler_lib().ref_sample_token(_pf(logits), logits.size, position, temperature, top_p, top_k, seed,
                                            C.cast(C.byref(token), _u32p))
    if rc != 0:
        raise RuntimeError(f"reference sampler failed with CUDA error {rc}")
    return token.value
