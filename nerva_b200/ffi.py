"""ctypes binding of libnerva_b200.so.

The struct classes are generated from include/nerva_b200_api.h at import time,
so the Python mirror cannot drift from the C declarations.  There is no CPU
fallback: loading fails loudly when the CUDA library has not been built.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(_HERE, "..", "include", "nerva_b200_api.h")
LIB_PATH = os.environ.get("NERVA_B200_LIB") or os.path.join(_HERE, "_lib", "libnerva_b200.so")

_SCALARS = {
    "uint8_t": C.c_uint8, "uint16_t": C.c_uint16, "uint32_t": C.c_uint32, "uint64_t": C.c_uint64,
    "int32_t": C.c_int32, "int64_t": C.c_int64, "float": C.c_float, "char": C.c_char,
}

structs: dict[str, type] = {}


def _field_type(ctype: str, pointer: bool):
    ctype = ctype.replace("const", "").strip()
    if pointer:
        if ctype == "char":
            return C.c_char_p
        return C.c_void_p  # typed access goes through numpy .ctypes.data
    if ctype in _SCALARS:
        return _SCALARS[ctype]
    return structs[ctype]


def _parse_header() -> None:
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for m in re.finditer(r"typedef struct (\w+) \{(.*?)\} \1;", text, flags=re.S):
        name, body = m.group(1), m.group(2)
        fields = []
        for line in body.split(";"):
            line = " ".join(line.split())
            if not line:
                continue
            fm = re.match(r"(.+?)\s*(\*?)\s*(\w+)$", line)
            ctype, star, fname = fm.group(1), fm.group(2), fm.group(3)
            pointer = bool(star) or ctype.endswith("*")
            fields.append((fname, _field_type(ctype.rstrip("* "), pointer)))
        structs[name] = type(name, (C.Structure,), {"_fields_": fields})


_parse_header()

TokenSlot = structs["NervaCudaSyntheticTokenSlot"]
ChainLayer = structs["NervaCudaHfDecodeChainLayer"]
WeightBlock = structs["NervaCudaHfDecodeSequenceWeightBlock"]
SamplerConfig = structs["NervaCudaHfDecodeSamplerConfig"]
SequenceRequest = structs["NervaCudaHfDecodeSequenceRequest"]
SequenceResult = structs["NervaCudaHfDecodeSequenceResult"]
LayoutPlanRequest = structs["NervaCudaHfDecodeSequenceLayoutPlanRequest"]
LayoutPlanResult = structs["NervaCudaHfDecodeSequenceLayoutPlanResult"]
CreateRequest = structs["NervaCudaHfDecodeSequenceSessionCreateRequest"]
CreateResult = structs["NervaCudaHfDecodeSequenceSessionCreateResult"]
ForkRequest = structs["NervaCudaHfDecodeSequenceSessionForkSharedWeightsRequest"]
RunRequest = structs["NervaCudaHfDecodeSequenceSessionRunRequest"]
StartRequest = structs["NervaCudaHfDecodeSequenceSessionStartRequest"]
AdvanceRequest = structs["NervaCudaHfDecodeSequenceSessionAdvanceRequest"]
ProjectionBenchRequest = structs["NervaCudaProjectionBenchRequest"]
ProjectionBenchResult = structs["NervaCudaProjectionBenchResult"]


def declared_functions() -> list[str]:
    """Names of every function the header declares."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nerva_(?:cuda|b200)_\w+)\s*\(", text)))


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m nerva_b200.build` (nvcc, sm_100a). "
            "There is no CPU fallback.")
    _lib = _bind(C.CDLL(LIB_PATH), reference_abi_only=False)
    return _lib


def load_abi_library(path: str) -> C.CDLL:
    """Another shared library that exports the reference's C ABI (the nerva_cuda_* entry points
    with the structs of include/nerva_b200_api.h), bound with the same signatures.  The session
    classes accept it through their `library` argument; the nerva_b200_* additions are not bound."""
    return _bind(C.CDLL(path), reference_abi_only=True)


def _bind(L: C.CDLL, reference_abi_only: bool) -> C.CDLL:
    P = C.POINTER
    vp = C.c_void_p
    sigs = {
        "nerva_cuda_hf_decode_sequence_plan_layout": [P(LayoutPlanRequest), P(LayoutPlanResult)],
        "nerva_cuda_hf_decode_sequence_session_create": [P(CreateRequest), P(CreateResult), P(vp)],
        "nerva_cuda_hf_decode_sequence_session_run": [P(RunRequest), P(SequenceResult)],
        "nerva_cuda_hf_decode_sequence_session_start": [P(StartRequest), P(SequenceResult)],
        "nerva_cuda_hf_decode_sequence_session_advance": [P(AdvanceRequest), P(SequenceResult)],
        "nerva_cuda_hf_decode_sequence_session_fork_shared_weights": [P(ForkRequest), P(CreateResult), P(vp)],
        "nerva_cuda_hf_decode_sequence_batch_advance_one": [
            P(structs["NervaCudaHfDecodeSequenceBatchAdvanceRequest"]),
            P(structs["NervaCudaHfDecodeSequenceBatchAdvanceResult"])],
        "nerva_cuda_hf_decode_sequence_session_destroy": [vp, P(CreateResult)],
        "nerva_cuda_hf_decode_sequence_u16": [P(SequenceRequest), P(SequenceResult)],
        "nerva_cuda_projection_bench": [P(ProjectionBenchRequest), P(ProjectionBenchResult)],
        "nerva_cuda_deepseek_router_route": [P(structs["NervaCudaDeepSeekRouterRouteRequest"]),
                                             P(structs["NervaCudaDeepSeekRouterRouteResult"])],
        "nerva_cuda_deepseek_mla_decode": [P(structs["NervaCudaDeepSeekMlaDecodeRequest"]),
                                           P(structs["NervaCudaDeepSeekMlaDecodeResult"])],
        "nerva_cuda_deepseek_moe_forward": [P(structs["NervaCudaDeepSeekMoeForwardRequest"]),
                                            P(structs["NervaCudaDeepSeekMoeForwardResult"])],
        "nerva_b200_session_set_engine": [vp, C.c_uint32],
        "nerva_b200_session_read_logits": [vp, vp, C.c_uint32],
        "nerva_b200_session_set_kv_block_table": [vp, vp, C.c_uint32],
        "nerva_b200_session_get_kv_block_table": [vp, vp, C.c_uint32],
        "nerva_b200_session_read_kv_row": [vp, C.c_uint32, C.c_uint32, C.c_uint32, vp, C.c_uint32],
        "nerva_b200_session_profile_steps": [vp, C.c_uint32, vp, vp, C.c_uint32],
        "nerva_b200_session_read_phase_cycles": [vp, vp, C.c_uint32],
        "nerva_b200_session_read_timeline": [vp, vp, C.c_uint32],
        "nerva_b200_session_create_sharded": [P(CreateRequest), P(structs["NervaB200ShardInfo"]), P(CreateResult),
                                              P(vp)],
        "nerva_b200_session_comm_handle": [vp, vp, C.c_uint32],
        "nerva_b200_session_attach_peers": [vp, vp, C.c_uint32],
        "nerva_b200_session_attach_loopback": [vp],
        "nerva_b200_projection": [vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                  P(C.c_uint64)],
        "nerva_b200_projection_sustained": [vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                            C.c_uint32, P(C.c_uint64)],
        "nerva_b200_gqa_decode_attention": [vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                            C.c_uint32, C.c_uint32, C.c_uint32, P(C.c_uint64)],
        "nerva_b200_gqa_decode_attention_sustained": [vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32,
                                                      C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                                      P(C.c_uint64)],
        "nerva_b200_gqa_decode_attention_static_scratch": [vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32,
                                                           C.c_uint32, C.c_uint32, C.c_uint32, vp],
        "nerva_b200_greedy_argmax": [vp, C.c_uint32, P(C.c_uint32)],
        "nerva_b200_sample_token": [vp, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_uint32, C.c_uint64,
                                    P(C.c_uint32)],
        "nerva_b200_synth_normal_bf16": [C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, vp],
        "nerva_b200_synth_normal_bf16_block": [C.c_uint64] * 7 + [C.c_float, vp],
    }
    if reference_abi_only:
        # another implementation of the reference's C ABI (same structs, same prototypes): bind the
        # nerva_cuda_* entry points it exports and nothing else
        for name, argtypes in sigs.items():
            if name.startswith("nerva_cuda_") and hasattr(L, name):
                fn = getattr(L, name)
                fn.argtypes = argtypes
                fn.restype = C.c_int
        return L
    for name, argtypes in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = argtypes
        fn.restype = None if name.startswith("nerva_b200_synth_normal_bf16") else C.c_int
    u32, u64, i64 = C.c_uint32, C.c_uint64, C.c_int64
    host = {  # host-side memory bookkeeping: name -> (restype, argtypes)
        "nerva_b200_static_arena_new": (vp, [u64]),
        "nerva_b200_static_arena_free": (None, [vp]),
        "nerva_b200_static_arena_reserve": (C.c_int, [vp, u64, u64, u32, P(u64)]),
        "nerva_b200_static_arena_used": (u64, [vp]),
        "nerva_b200_static_arena_remaining": (u64, [vp]),
        "nerva_b200_static_arena_restore": (C.c_int, [vp, u64]),
        "nerva_b200_kv_page_pool_new": (vp, [vp, u32, u32, u64, u64]),
        "nerva_b200_kv_page_pool_free": (None, [vp]),
        "nerva_b200_kv_page_pool_len": (u32, [vp]),
        "nerva_b200_kv_page_pool_free_pages": (u32, [vp]),
        "nerva_b200_kv_page_pool_allocate": (i64, [vp, u32, u32, u64]),
        "nerva_b200_kv_page_pool_retain": (C.c_int, [vp, u32, u64]),
        "nerva_b200_kv_page_pool_release": (C.c_int, [vp, u32, u64]),
        "nerva_b200_kv_page_pool_cache": (C.c_int, [vp, u32, C.c_char_p, u32, u32]),
        "nerva_b200_kv_page_pool_lookup_cached": (i64, [vp, C.c_char_p, u32]),
        "nerva_b200_kv_page_pool_retain_cached": (i64, [vp, C.c_char_p, u32, u64]),
        "nerva_b200_kv_page_pool_evict_cached": (C.c_int, [vp, u32]),
        "nerva_b200_kv_page_pool_page": (C.c_int, [vp, u32, P(structs["NervaB200KvPageInfo"])]),
    }
    for name, (restype, argtypes) in host.items():
        fn = getattr(L, name)
        fn.restype = restype
        fn.argtypes = argtypes
    L.nerva_b200_last_error.restype = C.c_char_p
    L.nerva_b200_last_error.argtypes = []
    return L


def last_error() -> str:
    return lib().nerva_b200_last_error().decode()
