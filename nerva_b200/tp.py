"""Tensor-parallel set-up of resident sessions: one process per GPU of one node.

The data path needs no collective library: the partial sums of the O and down projections and
the arg-max candidates travel between the GPUs inside the decode kernels (peer stores into
exchange buffers, bounded waits on arrival counters).  `torch.distributed` is used here only
as the host channel that carries the 64-byte buffer handles between the processes, and for
barriers around set-up.
"""
from __future__ import annotations

from . import ops, synth
from .session import CudaHfDecodeSequenceSession, SmokeStatus


def select_device(local_rank: int) -> None:
    """Makes GPU `local_rank` the current CUDA device of this process (all GPUs stay visible,
    which the peer mappings need)."""
    import torch
    torch.cuda.set_device(local_rank)
    torch.zeros(1, device=f"cuda:{local_rank}")  # creates the primary context the library will use


def connect(session: CudaHfDecodeSequenceSession, group=None) -> None:
    """Exchanges the exchange-buffer handles of all ranks and maps the peers' buffers."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    handles = [None] * world
    dist.all_gather_object(handles, session.comm_handle(), group=group)
    session.attach_peers(handles)
    dist.barrier(group)  # nobody launches a step before every rank has mapped every buffer


def create_session(cfg: synth.DecoderConfig, max_context_tokens: int, rank: int, world: int, full_checkpoint=None,
                   group=None) -> CudaHfDecodeSequenceSession:
    """Creates this rank's part of `cfg` (cut from full_checkpoint when given, else generated
    directly with the native generator) and connects it to the other ranks.  Dense models are
    cut tensor-parallel; models with sparse-MoE layers expert-parallel (every rank holds the
    whole model except its share of the routed and shared experts)."""
    if cfg.num_experts:
        if full_checkpoint is not None:
            shard = synth.expert_shard_checkpoint(full_checkpoint, rank, world)
        else:
            shard = synth.expert_checkpoint_shard(cfg, rank, world, block_fill=ops.synth_normal_bf16_block,
                                                  fill=ops.synth_normal_bf16)
    elif full_checkpoint is not None:
        shard = synth.shard_checkpoint(full_checkpoint, rank, world)
    else:
        shard = synth.dense_checkpoint_shard(cfg, rank, world, block_fill=ops.synth_normal_bf16_block,
                                             fill=ops.synth_normal_bf16)
    session = CudaHfDecodeSequenceSession(shard, max_context_tokens)
    if session.status != SmokeStatus.OK:
        raise RuntimeError(f"rank {rank}: sharded session create failed: {session.status} {session.error}")
    connect(session, group)
    return session
