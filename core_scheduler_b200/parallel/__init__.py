# SPDX-License-Identifier: Apache-2.0
"""Process-group plumbing: one process per GPU, torch.distributed (NCCL on GPUs, Gloo on CPUs)."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from .. import _C


def init_distributed(device: str = "cuda", timeout_s: float = 600.0):
    """Initialises torch.distributed from the torchrun environment and returns (comm, rank, world, local_rank).

    With WORLD_SIZE unset or 1 no process group is created and a size-1 communicator is returned.
    """
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world <= 1:
        return _C.get_comm_self(), 0, 1, local_rank
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if not dist.is_initialized():
        if device == "cuda":
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s),
                                    device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    pg = dist.distributed_c10d._get_default_group()
    comm = _C.comm_from_process_group(pg.group_name, device)
    return comm, rank, world, local_rank


class GPT2Trainer:
    """One training step of GPT-2 under a parallelisation strategy, assembled from the native pieces.

    mode "dp"   data parallel: every rank owns the model; gradient ranges are all-reduced in buckets while the
                backward pass continues, and the average is folded into the optimizer kernel (the reference's
                example/gpt2/gpt2_ddp.cpp does the same with NCCL buckets).
         "zero" data parallel with the sharded optimizer (fp32 master weights and AdamW moments split over the ranks):
                reduce-scatter + AdamW + all-gather in one kernel per bucket, overlapped with backward (GPUs).
         "tp"   tensor + sequence parallel over all ranks; every rank sees the whole batch (GPUs, or Gloo ranks).
    collectives "nvp2p" runs this library's peer-memory kernels (GPUs with peer access), "nccl" the library's.
    `max_tokens` (tensor parallel with "nvp2p" only) is the largest B*T of a step; it sizes the symmetric arena.
    On GPUs the parameters are fp32 masters with bf16 working copies and the step runs under bf16 autocast; on the
    CPU everything is fp32.

        comm, rank, world, local_rank = init_distributed("cuda")
        trainer = GPT2Trainer(gpt2_config("124M"), comm, world, local_rank, mode="dp")
        loss = trainer.step(input_ids, labels)          # core_scheduler_b200.Tensor handles
    """

    def __init__(self, config, comm=None, world: int = 1, local_rank: int = 0, mode: str = "dp", collectives: str = "nvp2p",
                 device: str = "cuda", lr: float = 3e-4, beta1: float = 0.9, beta2: float = 0.95, weight_decay: float = 0.1,
                 bucket_mb: float = 25.0, seed: int = 1234, scheduler=None, overlap_optimizer: bool = True,
                 max_tokens: int = 32 * 1024):
        import core_scheduler_b200 as cs

        assert mode in ("dp", "zero", "tp") and collectives in ("nvp2p", "nccl")
        self.config, self.world, self.mode, self.device = config, world, mode, device
        self.amp = device == "cuda"
        self.scheduler = scheduler or cs.DynamicScheduler(local_rank if device == "cuda" else 0, device=device)
        s = self.scheduler
        self.comm = comm if comm is not None else _C.get_comm_self()
        self.bucket = self.sync = self.symmetric = None
        peer = device == "cuda" and world > 1 and (collectives == "nvp2p" or mode == "zero")
        if peer:  # the same ranks, with collectives on peer-mapped symmetric memory
            pg = dist.distributed_c10d._get_default_group()
            self.comm = _C.comm_from_process_group(pg.group_name, "cuda", True)
        cs.manual_seed(seed)  # identical initial weights on every rank
        lp = dict(lp_dtype=torch.bfloat16) if self.amp else {}
        if mode == "tp" and world > 1:
            if peer:
                # gathered activations of every block are kept from forward to backward in symmetric buffers:
                # two [tokens, d] bf16 per block, plus the partial-product, gradient and classifier buffers
                rows_bytes = max_tokens * config.n_embd * 2
                arena = (2 * config.n_layer + 8) * rows_bytes + (256 << 20)
                # and this rank's gradient (fp32) and working-copy (bf16) arenas, so that the gradients of the
                # replicated parameters are reduced where the backward pass wrote them
                arena += (config.parameter_count() // world + 2 * config.padded_vocab_size * config.n_embd) * 6 + (64 << 20)
                self.symmetric = _C.create_symmetric_context(self.comm, int(arena))
            self.model = _C.TPGPT2(s, config, self.comm)
            # replicated parameters first: their gradients form one range (one all-reduce launch, one AdamW launch),
            # and so do the sharded ones
            replicated = self.model.replicated_parameters()
            if peer:
                self.flat = _C.flatten_symmetric(s, self.model, self.comm, first=replicated, unequal_shards=True)
            else:
                self.flat = _C.flatten_parameters(s, self.model, first=replicated, **lp)
        else:
            self.model = cs.GPT2(s, config)
            if peer:
                arena = config.parameter_count() * 6 + (256 << 20)  # fp32 gradients + bf16 copies + staging
                self.symmetric = _C.create_symmetric_context(self.comm, int(arena))
                self.flat = _C.flatten_symmetric(s, self.model, self.comm)
            else:
                self.flat = _C.flatten_parameters(s, self.model, **lp)
        if mode == "zero" and world > 1:
            assert peer, "the sharded optimizer runs on GPUs with peer access"
            self.optimizer = _C.ZeroAdamW(s, self.model, self.flat, self.comm, lr=lr, beta1=beta1, beta2=beta2,
                                          weight_decay=weight_decay)
            if overlap_optimizer:
                # every bucket of gradients is reduce-scattered, turned into an AdamW update of the blocks this rank owns
                # and all-gathered as bf16 working weights by one kernel, while the backward pass of the earlier layers runs
                self.bucket = cs.AllReduceBucket(int(bucket_mb * (1 << 20)), "sum")
                self.bucket.attach_sharded_optimizer(self.optimizer)
                self.sync = cs.GradientSync(self.comm, self.bucket, True)
        else:
            self.optimizer = cs.AdamW(s, self.model, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay, flat=self.flat)
            if world > 1:
                self.optimizer.set_grad_scale(1.0 / world)
            if world > 1 or overlap_optimizer:
                # gradients leave the backward pass in buckets; with overlap_optimizer each bucket's parameters
                # are updated right after its all-reduce, while the backward pass of the earlier layers runs
                self.bucket = cs.AllReduceBucket(int(bucket_mb * (1 << 20)), "sum")
                self.sync = cs.GradientSync(self.comm, self.bucket, True)
                if overlap_optimizer:
                    self.bucket.attach_optimizer(self.optimizer)
        s.synchronize()

    def check_device_status(self):
        """Raises when a kernel gave up on a bounded wait (a tensor-core pipeline barrier, a peer's flag): the numbers
        of such a step are meaningless. Synchronises the device; call it between steps, not inside a timed region."""
        if self.device != "cuda":
            return  # the CPU paths have no device-side waits
        torch.cuda.synchronize()
        for name, status in (("gemm", _C.gemm_status()), ("attention", _C.attention_status())):
            if status[0] != 0:
                raise RuntimeError(f"{name} kernel reported a timed-out wait: code={status[0]} kernel={status[1]} "
                                   f"block={status[2]} detail={status[3]}")
        if self.symmetric is not None:
            self.symmetric.check_status()

    def close(self):
        """Releases the symmetric arena in an orderly way: every rank drains its streams, all ranks meet, then the
        mappings (and the multicast binding) go. Call it on every rank before the process group is destroyed."""
        self.scheduler.synchronize()
        if self.symmetric is not None:
            torch.cuda.synchronize()
            if dist.is_initialized():
                dist.barrier()
            self.model = self.optimizer = self.flat = self.bucket = self.sync = None  # views into the arena
            self.symmetric = None
            self.comm.release_symmetric()

    def step(self, input_ids, labels):
        """Forward, backward (gradient communication overlapped), optimizer update; returns the loss handle."""
        import core_scheduler_b200 as cs

        s, m = self.scheduler, self.model
        if self.amp:
            with cs.autocast(s, torch.bfloat16):
                loss = m.forward_loss(s, input_ids, labels)
        else:
            loss = m.forward_loss(s, input_ids, labels)
        m.backward_loss(s, self.sync) if self.sync is not None else m.backward_loss(s)
        if self.bucket is not None:
            self.bucket.sync(s, self.comm)
        self.optimizer.step(s)
        self.optimizer.zero_grad(s)
        return loss
