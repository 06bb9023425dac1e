"""Host-side mirror of the reference's safe session wrappers.

Same names, argument meaning and status convention as the reference's FFI crate:
  CudaHfDecodeSequenceSession  crates/nerva-cuda/src/decode/hf_sequence/session/mod.rs
  CudaHfDecodeSequenceLoop     crates/nerva-cuda/src/decode/hf_sequence/session/stateful.rs:26-151
  SmokeStatus                  crates/nerva-cuda/src/decode/hf_sequence/status.rs:5-16
Everything below calls the C ABI of libnerva_b200.so with host buffers (numpy).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import ffi

CUDA_ERROR_NO_DEVICE = 100
CUDA_ERROR_NOT_SUPPORTED = 801
DTYPE_F16, DTYPE_BF16 = 0, 1
STRATEGY_GPU_RESIDENT, STRATEGY_GPU_STAGED = 1, 2


class SmokeStatus:
    OK = "ok"
    FAILED = "failed"
    UNAVAILABLE = "unavailable"


def _status(return_code: int, status: int, cuda_error: int, device_count: int) -> str:
    # status.rs:5-16: no device is "unavailable", not "failed"
    if return_code == 0 and status == 0:
        return SmokeStatus.OK
    if cuda_error == CUDA_ERROR_NO_DEVICE or (device_count == 0 and cuda_error != 0):
        return SmokeStatus.UNAVAILABLE
    return SmokeStatus.FAILED


def _ptr(a) -> int | None:
    return None if a is None else a.ctypes.data


@dataclass
class Summary:
    status: str
    tokens: list
    raw: object
    error: str = ""

    def __getattr__(self, name):  # counters of the C result struct
        return getattr(self.raw, name)


def greedy_sampler() -> "ffi.SamplerConfig":
    return ffi.SamplerConfig(temperature=0.0, top_p=1.0, top_k=0, reserved=0, seed=0)


def sampler_config(temperature: float = 0.7, top_p: float = 0.9, top_k: int = 0, seed: int = 0) -> "ffi.SamplerConfig":
    """Sampler of a request; the defaults are the reference's (hf_decode_sequence/sampler.cu:411-419)."""
    return ffi.SamplerConfig(temperature=temperature, top_p=top_p, top_k=top_k, reserved=0, seed=seed)


_LAYER_TENSORS = {
    "rms_attn": "rms_attn_weight", "rms_mlp": "rms_mlp_weight", "w_q": "w_q", "w_k": "w_k", "w_v": "w_v",
    "w_o": "w_o", "q_norm": "q_norm_weight", "k_norm": "k_norm_weight", "q_bias": "q_bias", "k_bias": "k_bias",
    "v_bias": "v_bias", "o_bias": "o_bias", "w_gate": "w_gate", "w_up": "w_up", "w_down": "w_down",
    "w_router": "w_router", "w_expert_gate_up": "w_expert_gate_up", "w_expert_down": "w_expert_down",
    "w_shared_expert_gate": "w_shared_expert_gate", "w_shared_expert_up": "w_shared_expert_up",
    "w_shared_expert_down": "w_shared_expert_down", "w_shared_expert_router": "w_shared_expert_router",
}


def chain_layers(checkpoint):
    """NervaCudaHfDecodeChainLayer array over a checkpoint's host tensors."""
    cfg = checkpoint.config
    arr = (ffi.ChainLayer * cfg.layers)()
    for i, entry in enumerate(checkpoint.layers):
        for key, fname in _LAYER_TENSORS.items():
            if key in entry:
                setattr(arr[i], fname, _ptr(entry[key]))
        if getattr(cfg, "kv_lora_rank", 0):
            arr[i].attention_kind = 2
            arr[i].deepseek_storage = 1  # bf16
            arr[i].deepseek_kv_lora_rank = cfg.kv_lora_rank
            arr[i].deepseek_qk_nope_head_dim = cfg.qk_nope_head_dim
            arr[i].deepseek_qk_rope_head_dim = cfg.qk_rope_head_dim
            arr[i].deepseek_v_head_dim = cfg.head_dim
        if cfg.num_experts and i >= getattr(cfg, "dense_layers", 0):
            arr[i].mlp_kind = 1
            arr[i].moe_intermediate = cfg.moe_intermediate
            arr[i].shared_expert_intermediate = cfg.shared_intermediate
            arr[i].num_experts = cfg.num_experts
            arr[i].experts_per_token = cfg.top_k
            arr[i].norm_topk_prob = int(cfg.norm_topk_prob)
    return arr


def hash_weight_blocks(blocks) -> int:
    """FNV-1a-64 over (block_id, block_version, offset_bytes, bytes, strategy), little endian
    (crates/nerva-cuda/src/decode/hf_sequence/weight_plan.rs:96-121)."""
    h = 0xCBF29CE484222325
    for b in blocks:
        for value, n in ((b.block_id, 8), (b.block_version, 8), (b.offset_bytes, 8), (b.bytes, 8), (b.strategy, 4)):
            for byte in range(n):
                h ^= (value >> (8 * byte)) & 0xFF
                h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def _upload_order(checkpoint) -> list:
    """Tensors in upload order: embeddings, per-layer tensors in arena order, final norm, lm_head."""
    tensors = [checkpoint.embeddings]
    order = ("rms_attn", "w_q", "q_norm", "w_k", "k_norm", "w_v", "w_o", "rms_mlp", "w_gate", "w_up", "w_down",
             "q_bias", "k_bias", "v_bias", "o_bias")
    cfg = checkpoint.config
    for entry in checkpoint.layers:
        if getattr(cfg, "kv_lora_rank", 0):
            # latent-attention layers (the reference's DeepSeek packing order,
            # hf_decode_sequence/deepseek/weights_pack.inc.cu:156-186,261-322): attention tensors, then the
            # dense MLP or router | shared expert | every expert's gate | every expert's up | every expert's down
            tensors += [entry[k] for k in ("rms_attn", "w_q", "w_kv_a", "kv_a_norm", "w_kv_b", "w_o", "rms_mlp")]
            if "w_router" in entry:
                tensors.append(entry["w_router"])
                tensors += [entry[k] for k in ("w_shared_expert_gate", "w_shared_expert_up", "w_shared_expert_down")
                            if k in entry]
                # -1: an expert-parallel rank holds fewer experts than the router has rows
                per_expert = entry["w_expert_gate_up"].reshape(-1, 2, cfg.moe_intermediate * cfg.hidden)
                tensors += [np.ascontiguousarray(per_expert[:, 0]).reshape(-1),
                            np.ascontiguousarray(per_expert[:, 1]).reshape(-1), entry["w_expert_down"]]
            else:
                tensors += [entry[k] for k in ("w_gate", "w_up", "w_down")]
            continue
        tensors += [entry[k] for k in order if k in entry]
    tensors += [checkpoint.final_norm, checkpoint.lm_head]
    return tensors


def write_weight_file(checkpoint, path: str, header_bytes: int = 0) -> None:
    """Writes the checkpoint's tensors back to back in upload order behind `header_bytes` of
    padding: a stand-in for the byte ranges of a safetensors shard that file-backed descriptors
    point at (crates/nerva-runtime/src/engine/hf_cuda_decode/file_backed/*)."""
    with open(path, "wb") as f:
        f.write(b"\0" * header_bytes)
        for t in _upload_order(checkpoint):
            f.write(np.ascontiguousarray(t).tobytes())


def weight_blocks(checkpoint, staged_every: int = 2, source_file: str | None = None, header_bytes: int = 0):
    """Descriptor table in upload order with contiguous offsets over the resident weight bytes.
    Blocks come from the host tensors, or (source_file) from byte ranges of a file laid out by
    write_weight_file, which the library reads through its pinned staging buffer
    (hf_decode_sequence/weights.cu:797-850).  Returns (array, objects to keep alive)."""
    tensors = _upload_order(checkpoint)
    arr = (ffi.WeightBlock * len(tensors))()
    path_bytes = source_file.encode() if source_file is not None else None
    offset = 0
    for i, t in enumerate(tensors):
        if path_bytes is None:
            arr[i].host_source = _ptr(t)
        else:
            arr[i].source_file = path_bytes
            arr[i].source_file_len = len(path_bytes)
            arr[i].file_offset_begin = header_bytes + offset
        arr[i].block_id = i + 1
        arr[i].block_version = 1
        arr[i].offset_bytes = offset
        arr[i].bytes = t.size * 2
        arr[i].strategy = STRATEGY_GPU_STAGED if staged_every and i % staged_every == 1 else STRATEGY_GPU_RESIDENT
        offset += t.size * 2
    arr._path_keepalive = path_bytes
    arr._tensor_keepalive = tensors  # re-packed copies (per-expert gate / up matrices) live as long as the table
    return arr


class CudaHfDecodeSequenceSession:
    """Owns one native session handle (create ... destroy)."""

    def __init__(self, checkpoint, max_context_tokens: int, use_descriptors: bool = False, dtype: int = DTYPE_BF16,
                 engine: int = 0, library=None, weight_file: str | None = None, weight_file_header: int = 0):
        """library: a handle from ffi.load_abi_library for another implementation of the same C ABI
        (default: this package's libnerva_b200.so).  weight_file: upload through descriptors that
        name byte ranges of this file (see write_weight_file) instead of host pointers."""
        cfg = checkpoint.config
        self._lib = library if library is not None else ffi.lib()
        self._own_library = library is None
        self.config = cfg
        self._keep = [checkpoint]
        layers = chain_layers(checkpoint)
        req = ffi.CreateRequest(
            dtype=dtype, hidden=cfg.hidden, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
            intermediate=cfg.intermediate, vocab_size=cfg.vocab, layer_count=cfg.layers,
            max_context_tokens=max_context_tokens, rms_eps=cfg.rms_eps, rope_theta=cfg.rope_theta,
            embeddings=_ptr(checkpoint.embeddings), layers=C.cast(layers, C.c_void_p),
            final_norm_weight=_ptr(checkpoint.final_norm), lm_head=_ptr(checkpoint.lm_head))
        if use_descriptors or weight_file is not None or getattr(cfg, "kv_lora_rank", 0):
            blocks = weight_blocks(checkpoint, source_file=weight_file, header_bytes=weight_file_header)
            self._keep.append(blocks)
            req.planned_weight_blocks = len(blocks)
            req.planned_weight_descriptor_count = len(blocks)
            req.planned_weight_descriptors = C.cast(blocks, C.c_void_p)
            req.planned_gpu_resident_blocks = sum(1 for b in blocks if b.strategy == STRATEGY_GPU_RESIDENT)
            req.planned_gpu_staged_blocks = sum(1 for b in blocks if b.strategy == STRATEGY_GPU_STAGED)
            req.planned_weight_bytes = sum(b.bytes for b in blocks)
            req.planned_gpu_resident_weight_bytes = sum(b.bytes for b in blocks if b.strategy == STRATEGY_GPU_RESIDENT)
            req.planned_gpu_staged_weight_bytes = sum(b.bytes for b in blocks if b.strategy == STRATEGY_GPU_STAGED)
            req.planned_weight_descriptor_hash = hash_weight_blocks(blocks)
        self.request = req
        self._handle = C.c_void_p()
        self.create_result = ffi.CreateResult()
        self.shard = getattr(checkpoint, "shard", None)
        if self.shard is not None:
            # a tensor- or expert-parallel rank: `checkpoint` holds this rank's slices (nerva_b200.synth.shard_checkpoint,
            # expert_shard_checkpoint)
            info = ffi.structs["NervaB200ShardInfo"](rank=self.shard.rank, world=self.shard.world,
                                                     full_vocab=self.shard.full_vocab,
                                                     vocab_offset=self.shard.vocab_offset,
                                                     mode=getattr(self.shard, "mode", 0))
            rc = self._lib.nerva_b200_session_create_sharded(C.byref(req), C.byref(info),
                                                             C.byref(self.create_result), C.byref(self._handle))
        else:
            rc = self._lib.nerva_cuda_hf_decode_sequence_session_create(C.byref(req), C.byref(self.create_result),
                                                                        C.byref(self._handle))
        r = self.create_result
        self.status = _status(rc, r.status, r.cuda_error, r.device_count)
        self.error = self._last_error()
        if self.status == SmokeStatus.OK and engine:
            if ffi.lib().nerva_b200_session_set_engine(self._handle, engine) != 0:
                raise RuntimeError("engine not available for this model")

    def _last_error(self) -> str:
        return ffi.last_error() if self._own_library else ""

    @classmethod
    def _from_handle(cls, parent, handle, result, status):
        self = cls.__new__(cls)
        self._lib = parent._lib
        self._own_library = parent._own_library
        self.config = parent.config
        self._keep = parent._keep
        self._handle = handle
        self.create_result = result
        self.status = status
        self.error = self._last_error()
        return self

    def create_summary(self):
        return self.create_result

    def raw_handle(self):
        return self._handle

    def fork_shared_weights(self) -> "CudaHfDecodeSequenceSession":
        req = ffi.ForkRequest(parent=self._handle, detailed_profile=0)
        handle, res = C.c_void_p(), ffi.CreateResult()
        rc = self._lib.nerva_cuda_hf_decode_sequence_session_fork_shared_weights(C.byref(req), C.byref(res),
                                                                                 C.byref(handle))
        return self._from_handle(self, handle, res, _status(rc, res.status, res.cuda_error, res.device_count))

    @staticmethod
    def batch_advance_one(sessions, target_block_tokens: int = 0, min_block_tokens: int = 0) -> Summary:
        """One token for every ready session that shares weights with the others (reference:
        CudaHfDecodeSequenceSession::batch_advance_one, decode/hf_sequence/session/request.rs:575-597).
        tokens[i] is sessions[i]'s token, or 0xFFFFFFFF when that session did not take part."""
        handles = (C.c_void_p * max(len(sessions), 1))(*[s.raw_handle() for s in sessions])
        tokens = np.full(max(len(sessions), 1), 0xFFFFFFFF, dtype=np.uint32)
        req = ffi.structs["NervaCudaHfDecodeSequenceBatchAdvanceRequest"](
            sessions=C.cast(handles, C.c_void_p), session_count=len(sessions),
            target_block_tokens=target_block_tokens, min_block_tokens=min_block_tokens,
            output_tokens=_ptr(tokens), output_token_capacity=len(sessions))
        out = ffi.structs["NervaCudaHfDecodeSequenceBatchAdvanceResult"]()
        library = sessions[0]._lib if sessions else ffi.lib()
        rc = library.nerva_cuda_hf_decode_sequence_batch_advance_one(C.byref(req), C.byref(out))
        return Summary(_status(rc, out.status, out.cuda_error, out.device_count), tokens[:len(sessions)].tolist(),
                       out, sessions[0]._last_error() if sessions else ffi.last_error())

    def run(self, prompt_tokens, steps: int, eos_token=None, sampler=None) -> Summary:
        prompt = np.ascontiguousarray(prompt_tokens, dtype=np.uint32)
        tokens = np.zeros(max(steps, 1), dtype=np.uint32)
        req = ffi.RunRequest(session=self._handle, steps=steps, seed_token=int(prompt[-1]) if prompt.size else 0,
                             prompt_tokens=_ptr(prompt), prompt_token_count=prompt.size,
                             has_eos_token=int(eos_token is not None), eos_token=eos_token or 0,
                             output_tokens=_ptr(tokens), output_token_capacity=steps,
                             sampler=sampler or greedy_sampler())
        out = ffi.SequenceResult()
        rc = self._lib.nerva_cuda_hf_decode_sequence_session_run(C.byref(req), C.byref(out))
        return Summary(_status(rc, out.status, out.cuda_error, out.device_count),
                       tokens[:out.observed_tokens].tolist(), out, self._last_error())

    def read_logits(self) -> np.ndarray:
        logits = np.empty(self.config.vocab, dtype=np.float32)
        if ffi.lib().nerva_b200_session_read_logits(self._handle, _ptr(logits), logits.size) != 0:
            raise RuntimeError("no logits available")
        return logits

    def set_kv_block_table(self, table) -> None:
        t = np.ascontiguousarray(table, dtype=np.uint32)
        if ffi.lib().nerva_b200_session_set_kv_block_table(self._handle, _ptr(t), t.size) != 0:
            raise ValueError("page table rejected (must be a permutation, set before start)")

    def kv_block_table(self) -> np.ndarray:
        pages = (self.create_result.max_context_tokens + 15) // 16
        t = np.zeros(pages, dtype=np.uint32)
        if ffi.lib().nerva_b200_session_get_kv_block_table(self._handle, _ptr(t), t.size) < 0:
            raise RuntimeError("page table read failed")
        return t

    def read_kv_row(self, layer: int, token: int, which: int) -> np.ndarray:
        row = np.zeros(self.config.kv_hidden, dtype=np.uint16)
        if ffi.lib().nerva_b200_session_read_kv_row(self._handle, layer, token, which, _ptr(row), row.size) != 0:
            raise RuntimeError("KV row read failed")
        return row

    PROFILE_BUCKETS = ("embed", "qkv", "attention", "o", "gate_up", "down", "lm_head", "sampling")

    def profile_steps(self, steps: int) -> dict:
        """Device nanoseconds per operator bucket over `steps` un-captured decode steps."""
        ns = np.zeros(8, dtype=np.uint64)
        launches = np.zeros(8, dtype=np.uint32)
        if ffi.lib().nerva_b200_session_profile_steps(self._handle, steps, _ptr(ns), _ptr(launches), 8) != 0:
            raise RuntimeError("profile_steps failed: " + ffi.last_error())
        return {name: {"ns": int(ns[i]), "launches_per_step": int(launches[i])}
                for i, name in enumerate(self.PROFILE_BUCKETS)}

    PHASES = ("qkv_prologue", "qkv", "barrier_qkv", "attention", "barrier_attention", "o_prologue", "o",
              "barrier_o", "gate_up_prologue", "gate_up", "barrier_gate_up", "down_prologue", "down",
              "barrier_down", "lm_head", "tail")

    def read_phase_cycles(self) -> dict:
        """Per-phase SM cycles of block 0 of the whole-step kernel since the last read
        (needs NERVA_B200_PHASE_PROFILE=1 in the environment when the session is created)."""
        cycles = np.zeros(16, dtype=np.uint64)
        if ffi.lib().nerva_b200_session_read_phase_cycles(self._handle, _ptr(cycles), 16) < 0:
            raise RuntimeError("phase cycles unavailable")
        return {name: int(c) for name, c in zip(self.PHASES, cycles)}

    def comm_handle(self) -> bytes:
        """64-byte inter-process handle of this tensor-parallel rank's exchange buffer."""
        buf = (C.c_uint8 * 64)()
        if ffi.lib().nerva_b200_session_comm_handle(self._handle, buf, 64) != 64:
            raise RuntimeError("no exchange buffer: " + ffi.last_error())
        return bytes(buf)

    def attach_peers(self, handles) -> None:
        """handles: the comm_handle() of every rank, in rank order."""
        blob = b"".join(handles)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        if ffi.lib().nerva_b200_session_attach_peers(self._handle, buf, len(handles)) != 0:
            raise RuntimeError("attach_peers failed: " + ffi.last_error())

    def attach_loopback(self) -> None:
        """Diagnostic: a tensor-parallel rank whose peers never answer (see the C header)."""
        if ffi.lib().nerva_b200_session_attach_loopback(self._handle) != 0:
            raise RuntimeError("attach_loopback failed")

    def read_timeline(self) -> np.ndarray:
        """%globaltimer stamps of the last step, shape [5 * layers + 1, 8] (launch order QKV, attention,
        O, gate/up, down per layer, then lm_head; columns: entry / after wait / after prologue / exit of
        the first block, then of the last block).  Needs NERVA_B200_TIMELINE=1 at create."""
        nodes = 5 * self.config.layers + 1
        stamps = np.zeros(nodes * 8, dtype=np.uint64)
        if ffi.lib().nerva_b200_session_read_timeline(self._handle, _ptr(stamps), stamps.size) < 0:
            raise RuntimeError("timeline unavailable")
        return stamps.reshape(nodes, 8)

    def destroy(self) -> None:
        if self._handle:
            self._lib.nerva_cuda_hf_decode_sequence_session_destroy(self._handle, None)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class CudaHfDecodeSequenceLoop:
    """start(prompt) then advance(steps) repeatedly; tokens never leave the device in between."""

    def __init__(self, session: CudaHfDecodeSequenceSession, eos_token=None):
        self.session = session
        self.eos_token = eos_token
        self.finished = False

    @classmethod
    def start(cls, session, prompt_tokens, eos_token=None, sampler=None):
        prompt = np.ascontiguousarray(prompt_tokens, dtype=np.uint32)
        req = ffi.StartRequest(session=session.raw_handle(), prompt_tokens=_ptr(prompt),
                               prompt_token_count=prompt.size, has_eos_token=int(eos_token is not None),
                               eos_token=eos_token or 0, sampler=sampler or greedy_sampler())
        out = ffi.SequenceResult()
        rc = session._lib.nerva_cuda_hf_decode_sequence_session_start(C.byref(req), C.byref(out))
        summary = Summary(_status(rc, out.status, out.cuda_error, out.device_count), [], out, session._last_error())
        return summary, (cls(session, eos_token) if summary.status == SmokeStatus.OK else None)

    def advance(self, steps: int) -> Summary:
        if self.finished:
            return Summary(SmokeStatus.FAILED, [], ffi.SequenceResult(), "loop is already finished")
        tokens = np.zeros(max(steps, 1), dtype=np.uint32)
        req = ffi.AdvanceRequest(session=self.session.raw_handle(), steps=steps, output_tokens=_ptr(tokens),
                                 output_token_capacity=steps)
        out = ffi.SequenceResult()
        rc = self.session._lib.nerva_cuda_hf_decode_sequence_session_advance(C.byref(req), C.byref(out))
        got = tokens[:min(out.observed_tokens, steps)].tolist()
        summary = Summary(_status(rc, out.status, out.cuda_error, out.device_count), got, out,
                          self.session._last_error())
        self.finished = summary.status == SmokeStatus.OK and (
            len(got) < steps or (self.eos_token is not None and bool(got) and got[-1] == self.eos_token))
        return summary
