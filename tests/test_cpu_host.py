"""Host-side logic of the library, checked without a GPU: the shared object loads and exports
what the header declares, the ABI layout equals the reference's, requests are validated before
any device call, layout integers, descriptor hashes, the arena and the KV page pool."""
import ctypes as C
import os

import numpy as np
import pytest

from tests.conftest import GOLDEN, _has_gpu
from nerva_b200 import ffi, ops, session, synth


def test_library_exports_every_declared_function(built_lib):
    names = ffi.declared_functions()
    assert len(names) >= 40
    for name in names:
        assert hasattr(built_lib, name), f"{name} is declared in the header but not exported"
    for required in ("nerva_cuda_hf_decode_sequence_plan_layout", "nerva_cuda_hf_decode_sequence_session_create",
                     "nerva_cuda_hf_decode_sequence_session_start", "nerva_cuda_hf_decode_sequence_session_advance",
                     "nerva_cuda_hf_decode_sequence_session_run", "nerva_cuda_hf_decode_sequence_session_destroy",
                     "nerva_cuda_hf_decode_sequence_session_fork_shared_weights", "nerva_cuda_hf_decode_sequence_u16",
                     "nerva_cuda_projection_bench"):
        assert required in names


def test_missing_library_is_an_error_not_a_fallback(monkeypatch):
    monkeypatch.setattr(ffi, "_lib", None)
    monkeypatch.setattr(ffi, "LIB_PATH", "/nonexistent/libnerva_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ffi.lib()


def test_struct_layout_equals_the_reference_header():
    """abi_layout.txt holds sizeof/offsetof printed by a C program compiled against the reference's
    nerva_cuda_api.h; the ctypes structures are generated from this repository's header."""
    expected = {}
    with open(os.path.join(GOLDEN, "abi_layout.txt")) as f:
        for line in f:
            key, value = line.split()
            expected[key] = int(value)
    checked = 0
    for name, cls in ffi.structs.items():
        if name not in expected:
            assert not name.startswith("NervaCuda"), f"{name} is missing from the golden layout"
            continue
        assert C.sizeof(cls) == expected[name], name
        for fname, _ in cls._fields_:
            assert getattr(cls, fname).offset == expected[f"{name}.{fname}"], f"{name}.{fname}"
            checked += 1
    assert checked == len(expected) - sum(1 for k in expected if "." not in k)
    assert C.sizeof(ffi.TokenSlot) == 40


def test_function_prototypes_equal_the_reference_header():
    """abi_prototypes.txt holds the reference header's prototypes (return type and parameter types,
    in order) of every nerva_cuda_* function this library exports."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    make_golden = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(make_golden)
    with open(ffi.HEADER) as f:
        ours = make_golden.prototypes(f.read())
    assert len(ours) >= 9
    with open(os.path.join(GOLDEN, "abi_prototypes.txt")) as f:
        expected = dict(line.rstrip("\n").split(" ", 1) for line in f if line.strip())
    assert sorted(expected) == sorted(ours)
    for name, proto in expected.items():
        assert ours[name] == proto, name


def test_synthetic_generator_native_and_numpy_twins_agree(built_lib):
    for tid, std, n in ((synth.T_EMBEDDINGS, 0.02, 5000), (synth.layer_tensor_id(3, synth.L_Q), 1.0, 777)):
        assert np.array_equal(ops.synth_normal_bf16(0, tid, n, std), synth.normal_bf16(0, tid, n, std))
    values = synth.bf16_to_f32(synth.normal_bf16(0, 99, 200000, 0.02))
    assert abs(float(values.mean())) < 2e-4 and abs(float(values.std()) - 0.02) < 2e-4
    ids = synth.prompt_ids(synth.TINY_QWEN3)
    assert ids.size == 64 and ids.max() < 32000
    perm = synth.permutation(1, synth.T_PAGE_TABLE, 100)
    assert sorted(perm.tolist()) == list(range(100))


def test_descriptor_hash_is_fnv1a64():
    assert session.hash_weight_blocks([]) == 0xCBF29CE484222325
    block = ffi.WeightBlock(block_id=0x61, block_version=0, offset_bytes=0, bytes=0, strategy=0)
    # FNV-1a over the byte 0x61 followed by 35 zero bytes, computed independently
    h = 0xCBF29CE484222325
    for byte in [0x61] + [0] * 35:
        h = ((h ^ byte) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    assert session.hash_weight_blocks([block]) == h
    # one byte of input is the published FNV-1a-64 test vector for "a"
    assert ((0xCBF29CE484222325 ^ 0x61) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF == 0xAF63DC4C8601EC8C


def _tiny_dims():
    return synth.TINY_QWEN3


def test_plan_layout_offsets_follow_pack_layer_order(built_lib, tiny_checkpoint):
    """embeddings | input | scratch | per layer {rms_attn, w_q, q_norm, w_k, k_norm, w_v, w_o, rms_mlp,
    w_gate, w_up, w_down} | final_norm | lm_head, in 16-bit elements
    (native/cuda/hf_decode_sequence/weights.cu:12-23,487-591)."""
    cfg = _tiny_dims()
    ck = tiny_checkpoint
    layers = session.chain_layers(ck)
    h, a, kv, d, i, v = cfg.hidden, cfg.attention_hidden, cfg.kv_hidden, cfg.head_dim, cfg.intermediate, cfg.vocab
    per_layer = h + a * h + d + kv * h + d + kv * h + h * a + h + 3 * i * h
    base = v * h + 2 * h
    for index in (0, 3):
        rc, out = ops.plan_layout(cfg, layers, layer_index=index)
        assert rc == 0 and out.status == 0
        start = base + index * per_layer
        assert out.rms_attn == start
        assert out.w_q == start + h
        assert out.q_norm == out.w_q + a * h
        assert out.w_k == out.q_norm + d
        assert out.k_norm == out.w_k + kv * h
        assert out.w_v == out.k_norm + d
        assert out.w_o == out.w_v + kv * h
        assert out.rms_mlp == out.w_o + h * a
        assert out.w_router == 0xFFFFFFFFFFFFFFFF  # dense layer: no router
        assert out.final_norm == base + cfg.layers * per_layer
        assert out.lm_head == out.final_norm + h
        # bytes of the reference's per-layer layout records (688 each), not of the arena
        assert out.layout_bytes == cfg.layers * 688
        # the resident weight byte space is the arena without the input|scratch gap
        assert out.resident_weight_bytes == (out.lm_head + v * h - 2 * h) * 2
    rc, out = ops.plan_layout(cfg, layers, layer_index=cfg.layers)
    assert rc == -1


def _create_request(cfg, ck, chain, **override):
    fields = dict(dtype=1, hidden=cfg.hidden, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
                  intermediate=cfg.intermediate, vocab_size=cfg.vocab, layer_count=cfg.layers, max_context_tokens=32,
                  rms_eps=cfg.rms_eps, rope_theta=cfg.rope_theta, embeddings=ck.embeddings.ctypes.data,
                  layers=C.cast(chain, C.c_void_p), final_norm_weight=ck.final_norm.ctypes.data,
                  lm_head=ck.lm_head.ctypes.data)
    fields.update(override)
    return ffi.CreateRequest(**fields)


@pytest.mark.parametrize("override", [
    dict(kv_heads=3),                 # heads % kv_heads != 0
    dict(kv_heads=16),                # more kv heads than heads
    dict(dtype=2),                    # f32 weights are not a session dtype
    dict(head_dim=63),                # odd head_dim with RoPE
    dict(hidden=0), dict(layer_count=0), dict(max_context_tokens=0),
    dict(embeddings=None), dict(lm_head=None), dict(layers=None),
])
def test_create_rejects_invalid_requests_before_touching_a_device(built_lib, tiny_checkpoint, override):
    """Argument errors are reported as failure stage 1 whether or not a device exists."""
    cfg = _tiny_dims()
    ck = tiny_checkpoint
    layers = session.chain_layers(ck)
    req = _create_request(cfg, ck, layers, **override)
    handle, out = C.c_void_p(), ffi.CreateResult()
    rc = built_lib.nerva_cuda_hf_decode_sequence_session_create(C.byref(req), C.byref(out), C.byref(handle))
    assert rc == -1 and out.status == -1 and not handle.value
    # session_api_lifecycle.inc.cu:15-27: stage 1 (invalid request), no CUDA error code, no device query
    assert out.failure_stage == 1 and out.cuda_error == 0 and out.device_count == 0
    assert out.hot_path_allocations == 0


def test_create_rejects_a_layer_without_weights(built_lib, tiny_checkpoint):
    cfg = _tiny_dims()
    ck = tiny_checkpoint
    layers = session.chain_layers(ck)
    layers[1].w_down = None
    req = _create_request(cfg, ck, layers)
    handle, out = C.c_void_p(), ffi.CreateResult()
    assert built_lib.nerva_cuda_hf_decode_sequence_session_create(C.byref(req), C.byref(out), C.byref(handle)) == -1
    assert out.failure_stage == 1 and out.cuda_error == 0


def test_null_arguments_are_rejected(built_lib):
    out = ffi.CreateResult()
    handle = C.c_void_p()
    assert built_lib.nerva_cuda_hf_decode_sequence_session_create(None, C.byref(out), C.byref(handle)) == -1
    seq = ffi.SequenceResult()
    assert built_lib.nerva_cuda_hf_decode_sequence_session_start(None, C.byref(seq)) == -1
    assert built_lib.nerva_cuda_hf_decode_sequence_session_advance(None, C.byref(seq)) == -1
    req = ffi.AdvanceRequest(session=None, steps=1)
    assert built_lib.nerva_cuda_hf_decode_sequence_session_advance(C.byref(req), C.byref(seq)) == -1
    assert seq.status == -1
    built_lib.nerva_cuda_hf_decode_sequence_session_destroy(None, None)  # refused, nothing to free


@pytest.mark.skipif(_has_gpu(), reason="needs a machine without a CUDA device")
def test_no_device_reads_as_unavailable_not_failed(built_lib, tiny_checkpoint):
    """crates/nerva-cuda/src/decode/hf_sequence/status.rs:5-16."""
    cfg = _tiny_dims()
    ck = tiny_checkpoint
    s = session.CudaHfDecodeSequenceSession(ck, 32)
    assert s.status == session.SmokeStatus.UNAVAILABLE
    with pytest.raises(RuntimeError):
        ops.projection(np.zeros(64, np.uint16), np.zeros(8, np.uint16), 8, 8)


# ---- StaticArena (crates/nerva-memory/src/tests/arena.rs) ----

def test_static_arena_reserves_stable_aligned_regions(built_lib):
    L = built_lib
    arena = L.nerva_b200_static_arena_new(1024)
    off = C.c_uint64(99)
    assert L.nerva_b200_static_arena_reserve(arena, 33, 1, 0, C.byref(off)) == 0 and off.value == 0
    assert L.nerva_b200_static_arena_reserve(arena, 64, 128, 0, C.byref(off)) == 0
    assert off.value == 128 and off.value % 128 == 0
    assert L.nerva_b200_static_arena_used(arena) == 192
    assert L.nerva_b200_static_arena_remaining(arena) == 1024 - 192
    assert L.nerva_b200_static_arena_reserve(arena, 1000, 1, 0, C.byref(off)) == -1  # exhausted, unchanged
    assert L.nerva_b200_static_arena_used(arena) == 192
    L.nerva_b200_static_arena_free(arena)


def test_static_arena_rejects_hot_path_reservation(built_lib):
    L = built_lib
    arena = L.nerva_b200_static_arena_new(1024)
    off = C.c_uint64(0)
    assert L.nerva_b200_static_arena_reserve(arena, 64, 64, 2, C.byref(off)) == -1
    assert L.nerva_b200_static_arena_used(arena) == 0
    assert L.nerva_b200_static_arena_reserve(arena, 64, 64, 1, C.byref(off)) == 0  # warm-up is allowed
    L.nerva_b200_static_arena_free(arena)


def test_static_arena_checkpoint_restore_rewinds_scratch(built_lib):
    L = built_lib
    arena = L.nerva_b200_static_arena_new(256)
    off = C.c_uint64(0)
    assert L.nerva_b200_static_arena_reserve(arena, 32, 8, 0, C.byref(off)) == 0
    checkpoint = L.nerva_b200_static_arena_used(arena)
    assert L.nerva_b200_static_arena_reserve(arena, 128, 16, 0, C.byref(off)) == 0
    assert L.nerva_b200_static_arena_used(arena) > checkpoint
    assert L.nerva_b200_static_arena_restore(arena, checkpoint) == 0
    assert L.nerva_b200_static_arena_used(arena) == checkpoint
    assert L.nerva_b200_static_arena_restore(arena, checkpoint + 1) == -1  # cannot move forward
    L.nerva_b200_static_arena_free(arena)


# ---- KvPagePool (crates/nerva-memory/src/tests/kv.rs:13-93) ----

def _page(L, pool, index):
    info = ffi.structs["NervaB200KvPageInfo"]()
    assert L.nerva_b200_kv_page_pool_page(pool, index, C.byref(info)) == 0
    return info


def test_kv_page_pool_preallocates_pages_in_the_arena(built_lib):
    L = built_lib
    arena = L.nerva_b200_static_arena_new(1024)
    pool = L.nerva_b200_kv_page_pool_new(arena, 4, 16, 128, 128)
    assert pool
    assert L.nerva_b200_kv_page_pool_len(pool) == 4 and L.nerva_b200_kv_page_pool_free_pages(pool) == 4
    assert L.nerva_b200_static_arena_used(arena) == 512
    assert [_page(L, pool, i).arena_offset for i in range(4)] == [0, 128, 256, 384]
    assert not L.nerva_b200_kv_page_pool_new(arena, 8, 16, 128, 128)  # 1024 more bytes do not fit
    L.nerva_b200_kv_page_pool_free(pool)
    L.nerva_b200_static_arena_free(arena)


def test_kv_page_pool_allocates_and_releases_pages_fifo(built_lib):
    L = built_lib
    arena = L.nerva_b200_static_arena_new(512)
    pool = L.nerva_b200_kv_page_pool_new(arena, 2, 16, 128, 64)
    handle = L.nerva_b200_kv_page_pool_allocate(pool, 32, 8, 7)
    assert handle == 0 and L.nerva_b200_kv_page_pool_free_pages(pool) == 1
    page = _page(L, pool, handle)
    assert (page.token_start, page.token_count, page.ref_count, page.last_use) == (32, 8, 1, 7)
    assert L.nerva_b200_kv_page_pool_allocate(pool, 0, 17, 8) == -2        # larger than a page: refused ...
    assert L.nerva_b200_kv_page_pool_free_pages(pool) == 1                 # ... and the page stays free
    assert L.nerva_b200_kv_page_pool_release(pool, handle, 8) == 0
    assert L.nerva_b200_kv_page_pool_free_pages(pool) == 2
    assert _page(L, pool, handle).ref_count == 0
    assert L.nerva_b200_kv_page_pool_release(pool, handle, 9) == -1        # double release
    # FIFO: the released page went to the back, so page 1 comes first, then page 0
    assert L.nerva_b200_kv_page_pool_allocate(pool, 0, 1, 10) == 1
    assert L.nerva_b200_kv_page_pool_allocate(pool, 0, 1, 11) == 0
    assert L.nerva_b200_kv_page_pool_allocate(pool, 0, 1, 12) == -1        # exhausted
    L.nerva_b200_kv_page_pool_free(pool)
    L.nerva_b200_static_arena_free(arena)


def test_kv_page_pool_caches_prefix_keys_and_retain_hits(built_lib):
    L = built_lib
    arena = L.nerva_b200_static_arena_new(512)
    pool = L.nerva_b200_kv_page_pool_new(arena, 2, 16, 128, 64)
    key = bytes([7] * 32)
    handle = L.nerva_b200_kv_page_pool_allocate(pool, 0, 16, 1)
    assert L.nerva_b200_kv_page_pool_cache(pool, handle, key, 3, 16) == 0
    assert L.nerva_b200_kv_page_pool_lookup_cached(pool, key, 3) == handle
    assert L.nerva_b200_kv_page_pool_lookup_cached(pool, key, 4) == -1      # other group id
    assert L.nerva_b200_kv_page_pool_release(pool, handle, 2) == 0
    assert L.nerva_b200_kv_page_pool_free_pages(pool) == 2
    assert L.nerva_b200_kv_page_pool_retain_cached(pool, key, 3, 3) == handle
    assert L.nerva_b200_kv_page_pool_free_pages(pool) == 1
    assert _page(L, pool, handle).ref_count == 1
    assert L.nerva_b200_kv_page_pool_evict_cached(pool, handle) == 1
    assert L.nerva_b200_kv_page_pool_lookup_cached(pool, key, 3) == -1
    assert L.nerva_b200_kv_page_pool_evict_cached(pool, handle) == 0
    L.nerva_b200_kv_page_pool_free(pool)
    L.nerva_b200_static_arena_free(arena)
