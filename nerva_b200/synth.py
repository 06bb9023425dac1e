"""Deterministic synthetic checkpoints and prompts (numpy twin of include/nerva_synth.h).

The reference's decode benchmarks run on random-init BF16 weights ~N(0, 0.02)
(seed 0), unit norm weights, and uniform prompt ids (seed 1).  Values are a pure
function of (seed, tensor id, element index), computed with integer arithmetic
plus one float32 multiply, so this module, the C header and the CUDA fill kernel
produce identical bits.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

T_EMBEDDINGS = 1
T_LM_HEAD = 2
T_PROMPT = 3
T_PAGE_TABLE = 4
T_ACTIVATION = 5
T_LAYER_BASE = 1000
L_WQ, L_WK, L_WV, L_WO, L_WGATE, L_WUP, L_WDOWN = 0, 1, 2, 3, 4, 5, 6
L_ROUTER, L_EXPERT_GATE_UP, L_EXPERT_DOWN = 7, 8, 9
L_SHARED_GATE, L_SHARED_UP, L_SHARED_DOWN = 10, 11, 12
L_Q_A, L_Q_B, L_KV_A, L_KV_B, L_K, L_V, L_Q = 13, 14, 15, 16, 17, 18, 19
L_SHARED_ROUTER = 20

BF16_ONE = 0x3F80


def layer_tensor_id(layer: int, slot: int) -> int:
    return T_LAYER_BASE + layer * 64 + slot


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def key(seed: int, tensor_id: int) -> np.uint64:
    with np.errstate(over="ignore"):
        return _mix64(np.uint64(seed) * GAMMA + np.uint64(tensor_id))


def u64(k: np.uint64, counter: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return _mix64(k + (counter.astype(np.uint64) + np.uint64(1)) * GAMMA)


def _fields16(h: np.ndarray) -> np.ndarray:
    m = np.uint64(0xFFFF)
    return ((h & m) + ((h >> np.uint64(16)) & m) + ((h >> np.uint64(32)) & m) + (h >> np.uint64(48))).astype(np.int64)


def normal_i32(seed: int, tensor_id: int, count: int, start: int = 0) -> np.ndarray:
    k = key(seed, tensor_id)
    idx = np.arange(start, start + count, dtype=np.uint64) * np.uint64(3)
    s = _fields16(u64(k, idx)) + _fields16(u64(k, idx + np.uint64(1))) + _fields16(u64(k, idx + np.uint64(2)))
    return (s - 6 * 65535).astype(np.int32)


def f32_to_bf16(values: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    rounded = ((bits.astype(np.uint64) + np.uint64(0x7FFF) + lsb) >> np.uint64(16)).astype(np.uint16)
    nan = ((bits & np.uint32(0x7F800000)) == np.uint32(0x7F800000)) & ((bits & np.uint32(0x007FFFFF)) != 0)
    return np.where(nan, ((bits >> np.uint32(16)) | np.uint32(1)).astype(np.uint16), rounded)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_f32(seed: int, tensor_id: int, count: int, std: float, start: int = 0) -> np.ndarray:
    scale = np.float32(np.float32(std) * np.float32(2.0 ** -16))
    return normal_i32(seed, tensor_id, count, start).astype(np.float32) * scale


def normal_bf16(seed: int, tensor_id: int, count: int, std: float, start: int = 0) -> np.ndarray:
    out = np.empty(count, dtype=np.uint16)
    chunk = 1 << 22
    for lo in range(0, count, chunk):
        n = min(chunk, count - lo)
        out[lo:lo + n] = f32_to_bf16(normal_f32(seed, tensor_id, n, std, start + lo))
    return out


def uniform_u32(seed: int, tensor_id: int, count: int, bound: int) -> np.ndarray:
    k = key(seed, tensor_id)
    return (u64(k, np.arange(count, dtype=np.uint64)) % np.uint64(bound)).astype(np.uint32)


def permutation(seed: int, tensor_id: int, count: int) -> np.ndarray:
    """Seeded Fisher-Yates shuffle of 0..count-1 (physical KV page ids)."""
    k = key(seed, tensor_id)
    draws = u64(k, np.arange(count, dtype=np.uint64))
    perm = list(range(count))
    for i in range(count - 1, 0, -1):
        j = int(draws[i] % np.uint64(i + 1))
        perm[i], perm[j] = perm[j], perm[i]
    return np.asarray(perm, dtype=np.uint32)


@dataclass
class DecoderConfig:
    name: str
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True
    prompt_tokens: int = 64
    decode_tokens: int = 32
    # softmax top-k MoE (mlp_kind 1); zero experts = dense SwiGLU
    num_experts: int = 0
    top_k: int = 0
    moe_intermediate: int = 0
    shared_intermediate: int = 0
    norm_topk_prob: bool = False
    dense_layers: int = 0          # leading layers that keep the dense MLP in a sparse-MoE model
    # DeepSeek multi-head latent attention (attention_kind 2); zero rank = ordinary attention.
    # heads * head_dim is the value width (head_dim = v_head_dim); shared experts are ungated.
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0

    @property
    def attention_hidden(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_hidden(self) -> int:
        return self.kv_heads * self.head_dim

    def active_weight_bytes_per_token(self) -> int:
        """Weight bytes one decoded token must stream in a latent-attention / sparse-MoE model: the
        attention projections, the dense or the routed + shared expert matrices it touches, lm_head."""
        h = self.hidden
        if self.kv_lora_rank:
            qdim = self.qk_nope_head_dim + self.qk_rope_head_dim
            attn = (self.heads * qdim * h + (self.kv_lora_rank + self.qk_rope_head_dim) * h
                    + self.heads * (self.qk_nope_head_dim + self.head_dim) * self.kv_lora_rank
                    + h * self.heads * self.head_dim)
        else:
            attn = (self.attention_hidden + 2 * self.kv_hidden) * h + h * self.attention_hidden
        dense = 3 * self.intermediate * h
        moe = self.num_experts * h + 3 * (self.top_k * self.moe_intermediate + self.shared_intermediate) * h
        moe_layers = max(0, self.layers - self.dense_layers) if self.num_experts else 0
        return 2 * (attn * self.layers + dense * (self.layers - moe_layers) + moe * moe_layers + self.vocab * h)

    def projection_bytes_per_token(self) -> int:
        """Weight bytes one decoded token must stream (2*N*K per projection)."""
        h = self.hidden
        per_layer = (self.attention_hidden + 2 * self.kv_hidden) * h + h * self.attention_hidden
        per_layer += 3 * self.intermediate * h
        return 2 * (per_layer * self.layers + self.vocab * h)


# DeepSeek-V2-Lite architecture: 27 layers, latent attention (rank 512, nope 128 / rope 64 / v 128),
# first layer dense (intermediate 10944), then 64 routed experts (top-6 softmax) + 2 shared experts
# of intermediate 1408 each (one ungated MLP of 2816).
DEEPSEEK_V2_LITE = DecoderConfig("deepseek-v2-lite", layers=27, hidden=2048, heads=16, kv_heads=16, head_dim=128,
                                 intermediate=10944, vocab=102400, rope_theta=1e4, qk_norm=False, prompt_tokens=1024,
                                 decode_tokens=128, num_experts=64, top_k=6, moe_intermediate=1408,
                                 shared_intermediate=2816, norm_topk_prob=False, dense_layers=1, kv_lora_rank=512,
                                 qk_nope_head_dim=128, qk_rope_head_dim=64)

TINY_QWEN3 = DecoderConfig("tiny-qwen3", layers=4, hidden=512, heads=8, kv_heads=2, head_dim=64,
                           intermediate=1536, vocab=32000, prompt_tokens=64, decode_tokens=32)
QWEN3_8B = DecoderConfig("qwen3-8b", layers=36, hidden=4096, heads=32, kv_heads=8, head_dim=128,
                         intermediate=12288, vocab=151936, prompt_tokens=512, decode_tokens=256)


@dataclass
class DenseCheckpoint:
    config: DecoderConfig
    embeddings: np.ndarray
    final_norm: np.ndarray
    lm_head: np.ndarray
    layers: list = field(default_factory=list)  # dict name -> uint16 array


def _attention_tensors(cfg: DecoderConfig, layer: int, seed: int, std: float, gen) -> dict:
    """Norm weights and attention projections of one layer (latent attention or Q/K/V/O)."""
    tid = lambda slot: layer_tensor_id(layer, slot)  # noqa: E731
    ones_h = np.full(cfg.hidden, BF16_ONE, dtype=np.uint16)
    if cfg.kv_lora_rank:
        qdim = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
        return {
            "rms_attn": ones_h.copy(),
            "rms_mlp": ones_h.copy(),
            "w_q": gen(seed, tid(L_Q), cfg.heads * qdim * cfg.hidden, std),
            "w_kv_a": gen(seed, tid(L_KV_A), (cfg.kv_lora_rank + cfg.qk_rope_head_dim) * cfg.hidden, std),
            "kv_a_norm": np.full(cfg.kv_lora_rank, BF16_ONE, dtype=np.uint16),
            "w_kv_b": gen(seed, tid(L_KV_B), cfg.heads * (cfg.qk_nope_head_dim + cfg.head_dim) * cfg.kv_lora_rank, std),
            "w_o": gen(seed, tid(L_WO), cfg.hidden * cfg.attention_hidden, std),
        }
    entry = {
        "rms_attn": ones_h.copy(),
        "rms_mlp": ones_h.copy(),
        "w_q": gen(seed, tid(L_WQ), cfg.attention_hidden * cfg.hidden, std),
        "w_k": gen(seed, tid(L_WK), cfg.kv_hidden * cfg.hidden, std),
        "w_v": gen(seed, tid(L_WV), cfg.kv_hidden * cfg.hidden, std),
        "w_o": gen(seed, tid(L_WO), cfg.hidden * cfg.attention_hidden, std),
    }
    if cfg.qk_norm:
        ones_d = np.full(cfg.head_dim, BF16_ONE, dtype=np.uint16)
        entry["q_norm"] = ones_d.copy()
        entry["k_norm"] = ones_d.copy()
    return entry


def dense_checkpoint(cfg: DecoderConfig, seed: int = 0, std: float = 0.02, fill=None) -> DenseCheckpoint:
    """Random-init BF16 checkpoint.  `fill(seed, tensor_id, count, std)` may be a
    native generator (same bits, multi-threaded) for the full-size models."""
    gen = fill or normal_bf16
    ones_h = np.full(cfg.hidden, BF16_ONE, dtype=np.uint16)
    ck = DenseCheckpoint(
        cfg,
        embeddings=gen(seed, T_EMBEDDINGS, cfg.vocab * cfg.hidden, std),
        final_norm=ones_h.copy(),
        lm_head=gen(seed, T_LM_HEAD, cfg.vocab * cfg.hidden, std),
    )
    for layer in range(cfg.layers):
        tid = lambda slot: layer_tensor_id(layer, slot)  # noqa: E731
        entry = _attention_tensors(cfg, layer, seed, std, gen)
        if cfg.num_experts == 0 or layer < cfg.dense_layers:
            entry["w_gate"] = gen(seed, tid(L_WGATE), cfg.intermediate * cfg.hidden, std)
            entry["w_up"] = gen(seed, tid(L_WUP), cfg.intermediate * cfg.hidden, std)
            entry["w_down"] = gen(seed, tid(L_WDOWN), cfg.hidden * cfg.intermediate, std)
        else:
            mi, e = cfg.moe_intermediate, cfg.num_experts
            entry["w_router"] = gen(seed, tid(L_ROUTER), e * cfg.hidden, std)
            entry["w_expert_gate_up"] = gen(seed, tid(L_EXPERT_GATE_UP), e * 2 * mi * cfg.hidden, std)
            entry["w_expert_down"] = gen(seed, tid(L_EXPERT_DOWN), e * cfg.hidden * mi, std)
            if cfg.shared_intermediate:
                si = cfg.shared_intermediate
                entry["w_shared_expert_gate"] = gen(seed, tid(L_SHARED_GATE), si * cfg.hidden, std)
                entry["w_shared_expert_up"] = gen(seed, tid(L_SHARED_UP), si * cfg.hidden, std)
                entry["w_shared_expert_down"] = gen(seed, tid(L_SHARED_DOWN), cfg.hidden * si, std)
                if not cfg.kv_lora_rank:  # DeepSeek shared experts are always on: no router row
                    entry["w_shared_expert_router"] = gen(seed, tid(L_SHARED_ROUTER), cfg.hidden, std)
        ck.layers.append(entry)
    return ck


@dataclass
class ShardInfo:
    rank: int
    world: int
    full_vocab: int
    vocab_offset: int
    mode: int = 0  # 0: tensor parallel, 1: expert parallel


def shard_config(cfg: DecoderConfig, world: int) -> DecoderConfig:
    """Dimensions one tensor-parallel rank holds: its share of the query heads, KV heads,
    intermediate size and lm_head rows; hidden size, head_dim and layer count stay."""
    import dataclasses
    if cfg.num_experts:
        raise ValueError("tensor parallel sharding covers dense layers")
    for name, value in (("heads", cfg.heads), ("kv_heads", cfg.kv_heads), ("intermediate", cfg.intermediate),
                        ("vocab", cfg.vocab)):
        if value % world:
            raise ValueError(f"{name}={value} is not divisible by {world} ranks")
    return dataclasses.replace(cfg, name=f"{cfg.name} shard 1/{world}", heads=cfg.heads // world,
                               kv_heads=cfg.kv_heads // world, intermediate=cfg.intermediate // world,
                               vocab=cfg.vocab // world)


def _numpy_block(seed, tensor_id, full_cols, row_begin, rows, col_begin, cols, std):
    full = normal_bf16(seed, tensor_id, (row_begin + rows) * full_cols, std).reshape(-1, full_cols)
    return np.ascontiguousarray(full[row_begin:row_begin + rows, col_begin:col_begin + cols]).reshape(-1)


def dense_checkpoint_shard(cfg: DecoderConfig, rank: int, world: int, seed: int = 0, std: float = 0.02,
                           block_fill=None, fill=None) -> DenseCheckpoint:
    """Rank `rank`'s slice of dense_checkpoint(cfg): QKV, gate/up and lm_head by rows, O and down
    by columns, norms and the embedding table whole.  Generated directly (no full model in
    memory) with the same bits as the slices of the full tensors.  The result carries
    `.shard` (ShardInfo) and `.config` (the local dimensions)."""
    local = shard_config(cfg, world)
    block = block_fill or _numpy_block
    gen = fill or normal_bf16
    h, d = cfg.hidden, cfg.head_dim
    ah, kvh, inter = cfg.attention_hidden, cfg.kv_hidden, cfg.intermediate
    lah, lkvh, linter = local.attention_hidden, local.kv_hidden, local.intermediate
    ones_h = np.full(h, BF16_ONE, dtype=np.uint16)
    ones_d = np.full(d, BF16_ONE, dtype=np.uint16)
    ck = DenseCheckpoint(
        local,
        embeddings=gen(seed, T_EMBEDDINGS, cfg.vocab * h, std),
        final_norm=ones_h.copy(),
        lm_head=block(seed, T_LM_HEAD, h, rank * local.vocab, local.vocab, 0, h, std),
    )
    ck.shard = ShardInfo(rank, world, cfg.vocab, rank * local.vocab)
    for layer in range(cfg.layers):
        tid = lambda slot: layer_tensor_id(layer, slot)  # noqa: E731
        entry = {
            "rms_attn": ones_h.copy(),
            "rms_mlp": ones_h.copy(),
            "w_q": block(seed, tid(L_WQ), h, rank * lah, lah, 0, h, std),
            "w_k": block(seed, tid(L_WK), h, rank * lkvh, lkvh, 0, h, std),
            "w_v": block(seed, tid(L_WV), h, rank * lkvh, lkvh, 0, h, std),
            "w_o": block(seed, tid(L_WO), ah, 0, h, rank * lah, lah, std),
            "w_gate": block(seed, tid(L_WGATE), h, rank * linter, linter, 0, h, std),
            "w_up": block(seed, tid(L_WUP), h, rank * linter, linter, 0, h, std),
            "w_down": block(seed, tid(L_WDOWN), inter, 0, h, rank * linter, linter, std),
        }
        if cfg.qk_norm:
            entry["q_norm"] = ones_d.copy()
            entry["k_norm"] = ones_d.copy()
        ck.layers.append(entry)
    return ck


def shard_checkpoint(full: DenseCheckpoint, rank: int, world: int) -> DenseCheckpoint:
    """The same slices cut out of a full checkpoint that is already in memory."""
    cfg = full.config
    local = shard_config(cfg, world)
    h = cfg.hidden
    lah, lkvh, linter = local.attention_hidden, local.kv_hidden, local.intermediate

    def rows(t, cols, begin, count):
        return np.ascontiguousarray(t.reshape(-1, cols)[begin:begin + count]).reshape(-1)

    def cols_of(t, full_cols, begin, count):
        return np.ascontiguousarray(t.reshape(-1, full_cols)[:, begin:begin + count]).reshape(-1)

    ck = DenseCheckpoint(local, embeddings=full.embeddings, final_norm=full.final_norm,
                         lm_head=rows(full.lm_head, h, rank * local.vocab, local.vocab))
    ck.shard = ShardInfo(rank, world, cfg.vocab, rank * local.vocab)
    for entry in full.layers:
        out = {k: v for k, v in entry.items() if k in ("rms_attn", "rms_mlp", "q_norm", "k_norm", "o_bias")}
        out["w_q"] = rows(entry["w_q"], h, rank * lah, lah)
        out["w_k"] = rows(entry["w_k"], h, rank * lkvh, lkvh)
        out["w_v"] = rows(entry["w_v"], h, rank * lkvh, lkvh)
        out["w_o"] = cols_of(entry["w_o"], cfg.attention_hidden, rank * lah, lah)
        out["w_gate"] = rows(entry["w_gate"], h, rank * linter, linter)
        out["w_up"] = rows(entry["w_up"], h, rank * linter, linter)
        out["w_down"] = cols_of(entry["w_down"], cfg.intermediate, rank * linter, linter)
        for name, width in (("q_bias", lah), ("k_bias", lkvh), ("v_bias", lkvh)):
            if name in entry:
                out[name] = np.ascontiguousarray(entry[name][rank * width:(rank + 1) * width])
        ck.layers.append(out)
    return ck


def expert_shard_config(cfg: DecoderConfig, world: int) -> DecoderConfig:
    """Dimensions one expert-parallel rank holds: everything except the routed experts (num_experts /
    world consecutive ones per sparse layer; num_experts itself stays the layer's total, the router
    is whole) and the shared expert, of which it holds a 1 / world slice of the intermediate size."""
    import dataclasses
    if not cfg.num_experts:
        raise ValueError("expert parallel needs sparse layers")
    if cfg.num_experts % world or cfg.shared_intermediate % (8 * world):
        raise ValueError(f"{cfg.num_experts} experts / shared intermediate {cfg.shared_intermediate} do not split "
                         f"over {world} ranks")
    if (cfg.layers - cfg.dense_layers) % 2:
        raise ValueError("expert parallel needs an even number of sparse layers")
    return dataclasses.replace(cfg, name=f"{cfg.name} experts 1/{world}",
                               shared_intermediate=cfg.shared_intermediate // world)


def _expert_slices(entry: dict, cfg: DecoderConfig, rank: int, world: int, cut) -> dict:
    """The sparse-MLP tensors of one layer as rank `rank` holds them.  cut(name, full_cols, row_begin,
    rows, col_begin, cols) returns that block of the full tensor `name` seen as a matrix."""
    h, mi, si = cfg.hidden, cfg.moe_intermediate, cfg.shared_intermediate
    local_e, local_si = cfg.num_experts // world, si // world
    out = {"w_router": entry["w_router"] if entry is not None else None}
    out["w_expert_gate_up"] = cut("w_expert_gate_up", 2 * mi * h, rank * local_e, local_e, 0, 2 * mi * h)
    out["w_expert_down"] = cut("w_expert_down", h * mi, rank * local_e, local_e, 0, h * mi)
    if si:
        out["w_shared_expert_gate"] = cut("w_shared_expert_gate", h, rank * local_si, local_si, 0, h)
        out["w_shared_expert_up"] = cut("w_shared_expert_up", h, rank * local_si, local_si, 0, h)
        out["w_shared_expert_down"] = cut("w_shared_expert_down", si, 0, h, rank * local_si, local_si)
    return out


def expert_shard_checkpoint(full: DenseCheckpoint, rank: int, world: int) -> DenseCheckpoint:
    """Rank `rank`'s part of a sparse-MoE checkpoint under expert parallel, cut out of the full
    checkpoint: dense tensors are shared with it (no copy), expert tensors are slices."""
    cfg = full.config
    local = expert_shard_config(cfg, world)
    ck = DenseCheckpoint(local, embeddings=full.embeddings, final_norm=full.final_norm, lm_head=full.lm_head)
    ck.shard = ShardInfo(rank, world, cfg.vocab, 0, mode=1)
    for entry in full.layers:
        if "w_router" not in entry:
            ck.layers.append(entry)
            continue

        def cut(name, full_cols, row_begin, rows, col_begin, cols, entry=entry):
            m = entry[name].reshape(-1, full_cols)[row_begin:row_begin + rows, col_begin:col_begin + cols]
            return np.ascontiguousarray(m).reshape(-1)

        out = {k: v for k, v in entry.items() if not k.startswith("w_expert") and not k.startswith("w_shared_expert")}
        out.update({k: v for k, v in _expert_slices(entry, cfg, rank, world, cut).items() if v is not None})
        if "w_shared_expert_router" in entry:
            out["w_shared_expert_router"] = entry["w_shared_expert_router"]
        ck.layers.append(out)
    return ck


def expert_checkpoint_shard(cfg: DecoderConfig, rank: int, world: int, seed: int = 0, std: float = 0.02,
                            block_fill=None, fill=None) -> DenseCheckpoint:
    """The same part generated directly (the full model's expert tensors never exist in memory),
    with the same bits as the slices of dense_checkpoint(cfg)."""
    local = expert_shard_config(cfg, world)
    block = block_fill or _numpy_block
    gen = fill or normal_bf16
    h = cfg.hidden
    ck = DenseCheckpoint(local, embeddings=gen(seed, T_EMBEDDINGS, cfg.vocab * h, std),
                         final_norm=np.full(h, BF16_ONE, dtype=np.uint16),
                         lm_head=gen(seed, T_LM_HEAD, cfg.vocab * h, std))
    ck.shard = ShardInfo(rank, world, cfg.vocab, 0, mode=1)
    names = {"w_expert_gate_up": L_EXPERT_GATE_UP, "w_expert_down": L_EXPERT_DOWN, "w_shared_expert_gate": L_SHARED_GATE,
             "w_shared_expert_up": L_SHARED_UP, "w_shared_expert_down": L_SHARED_DOWN}
    for layer in range(cfg.layers):
        tid = lambda slot: layer_tensor_id(layer, slot)  # noqa: E731
        entry = _attention_tensors(cfg, layer, seed, std, gen)
        if layer < cfg.dense_layers:
            entry["w_gate"] = gen(seed, tid(L_WGATE), cfg.intermediate * h, std)
            entry["w_up"] = gen(seed, tid(L_WUP), cfg.intermediate * h, std)
            entry["w_down"] = gen(seed, tid(L_WDOWN), h * cfg.intermediate, std)
            ck.layers.append(entry)
            continue

        def cut(name, full_cols, row_begin, rows, col_begin, cols, layer=layer):
            return block(seed, layer_tensor_id(layer, names[name]), full_cols, row_begin, rows, col_begin, cols, std)

        entry["w_router"] = gen(seed, tid(L_ROUTER), cfg.num_experts * h, std)
        entry.update({k: v for k, v in _expert_slices(None, cfg, rank, world, cut).items() if v is not None})
        if cfg.shared_intermediate and not cfg.kv_lora_rank:
            entry["w_shared_expert_router"] = gen(seed, tid(L_SHARED_ROUTER), h, std)
        ck.layers.append(entry)
    return ck


def prompt_ids(cfg: DecoderConfig, seed: int = 1, count: int | None = None) -> np.ndarray:
    return uniform_u32(seed, T_PROMPT, cfg.prompt_tokens if count is None else count, cfg.vocab)
