#!/usr/bin/env python
"""Benchmark of the fused layer kernels: the token-sharded transformer-block chain.

A "step" is one forward + backward pass of the non-GEMM chain of a transformer
block over one batch of synthetic tokens (batch 8 x seq 4096, d_model 4096,
d_ff 16384, vocab 32000, bf16 storage, fp32 arithmetic):

    forward   sort token ids -> embedding gather + positional encoding
              -> LN1(x + attn_out) -> bias + ReLU on the d_ff activation -> LN2(y1 + ff_out)
    backward  LN2 bwd -> ReLU bwd (+ bias grad) -> LN1 bwd with the gradient
              residual add folded in -> embedding-table scatter-add
              -> (N > 1) all-reduce of the gamma/beta/bias and table gradients

Random-normal tensors stand in for the GEMM outputs (attn_out, the d_ff
pre-activation, ff_out and the matching upstream gradients); they live on the
device, as the reference's own intermediate buffers do.  Token rows are split
evenly over the N ranks (strong scaling: the global batch is fixed).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference ...                     # the reference's own CUDA kernels

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

BATCH, SEQ, D_MODEL, D_FF, VOCAB = 8, 4096, 4096, 16384, 32000
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


# --------------------------------------------------------------------------- utilities
def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def zipf_ids(rng, n, vocab, s=1.1):
    """Bounded Zipf over [0, vocab), hot ids spread over the table by a fixed permutation."""
    p = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    p /= p.sum()
    ids = rng.choice(vocab, size=n, p=p)
    perm = np.random.Generator(np.random.Philox(key=77)).permutation(vocab)
    return perm[ids].astype(np.int32)


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, device_index: int, period_s: float = 0.002):
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self._nv = pynvml
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    _NAMES = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self._NAMES.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            time.sleep(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": round(max(self.power), 1) if self.power else None}


class Dist:
    def __init__(self):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.active = self.world > 1

    def init(self):
        torch.cuda.set_device(self.local_rank)
        if self.active:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist

    def barrier(self):
        if self.active:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_float(self, v: float) -> float:
        if not self.active:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def finish(self):
        if self.active:
            self.dist.destroy_process_group()


class LaggedReadback:
    """Device-to-host read of every step's result, consumed one step late: the copy of step i's result is
    queued behind step i's kernels, and the host waits for it (and reads it) only after it has queued step
    i+1 -- what a training loop that logs its loss does, so the GPU never idles while the host catches up.
    Every result is still copied and read inside the timed region; drain() takes the last one."""

    def __init__(self, n):
        self.bufs = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)]
        self.events = [torch.cuda.Event(), torch.cuda.Event()]
        self.count, self.pending = 0, False

    def push(self, src):
        k = self.count & 1
        self.bufs[k].copy_(src, non_blocking=True)
        self.events[k].record()
        self.count += 1
        previous = None
        if self.pending:
            self.events[k ^ 1].synchronize()
            previous = float(self.bufs[k ^ 1][0])
        self.pending = True
        return previous

    def drain(self):
        if not self.pending:
            return None
        k = (self.count - 1) & 1
        self.events[k].synchronize()
        self.pending = False
        return float(self.bufs[k][0])


# --------------------------------------------------------------------------- the chain (this library)
class Chain:
    """Buffers and the step of the block chain for `tokens` local token rows."""

    OPS = ["sort_tokens", "embed_gather_pe", "ln1_fwd", "relu_fwd", "ln2_fwd",
           "ln2_bwd", "relu_bwd", "ln1_bwd", "embed_scatter", "allreduce"]

    def __init__(self, tokens, seq, d, f, vocab, dtype, seed, dist: Dist, exchange="peer", clear="incremental",
                 split_push=True, plan_after_gather=True, first_position=0, seq_total=None):
        from dl_cuda_b200 import capi, ops
        global allreduce_param_grads
        from dl_cuda_b200.sharding import allreduce_param_grads
        self.capi, self.ops, self.lib = capi, ops, capi.lib()
        self.T, self.S, self.D, self.F, self.V = tokens, seq, d, f, vocab
        self.dist = dist
        self.dtype = dtype
        self.code = capi.BF16 if dtype == torch.bfloat16 else capi.F32
        self.e = 2 if dtype == torch.bfloat16 else 4
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device=dev)
        g.manual_seed(seed)

        def randn(*shape, scale=1.0):
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(dtype)

        T, D, F, V = tokens, d, f, vocab
        # parameters (replicated on every rank)
        gp = torch.Generator(device=dev)
        gp.manual_seed(4242)
        self.table = (torch.randn(V, D, generator=gp, device=dev) * 0.02).to(dtype)
        # this rank's rows of the positional-encoding table (all of it unless the ranks split the positions)
        self.pe = ops.pe_table(seq_total or seq, D)[first_position:first_position + seq].contiguous().to(dev)
        self.gamma1 = torch.rand(D, generator=gp, device=dev) + 0.5
        self.beta1 = torch.randn(D, generator=gp, device=dev) * 0.1
        self.gamma2 = torch.rand(D, generator=gp, device=dev) + 0.5
        self.beta2 = torch.randn(D, generator=gp, device=dev) * 0.1
        self.bias1 = torch.randn(F, generator=gp, device=dev) * 0.1
        # token ids: pinned host copy (the only per-step host input) and device copy
        # Two batches of ids, taken in turn: a step then meets a table gradient whose non-zero rows are
        # those of ANOTHER batch, as in training (with one batch repeated, nothing would ever need clearing).
        rng = np.random.Generator(np.random.Philox(key=seed))
        self.h_id_sets = [torch.from_numpy(zipf_ids(rng, T, V)).pin_memory() for _ in range(2)]
        self.id_sets = [h.to(dev) for h in self.h_id_sets]
        self.h_ids, self.ids = self.h_id_sets[0], self.id_sets[0]
        self.step_no = 0
        # stand-ins for GEMM outputs
        self.attn_out, self.ff_out = randn(T, D), randn(T, D)
        self.ff_pre = randn(T, F)
        self.dy, self.d_ff_in = randn(T, D), randn(T, D)
        self.d_act = randn(T, F)
        # activations, caches, gradients
        e = lambda *s: torch.empty(*s, device=dev, dtype=dtype)
        self.x0, self.y1, self.xhat1, self.y2, self.xhat2 = e(T, D), e(T, D), e(T, D), e(T, D), e(T, D)
        self.inv1 = torch.empty(T, device=dev)
        self.inv2 = torch.empty(T, device=dev)
        self.act = e(T, F)
        self.mask = torch.empty(self.lib.dlb_act_cache_bytes(capi.RELU, T * F, self.code), dtype=torch.uint8, device=dev)
        self.dx2, self.dx1 = e(T, D), e(T, D)
        self.d_pre = e(T, F)
        # every small parameter gradient sits in one buffer: one all-reduce
        self.small_grads = torch.empty(4 * D + F, device=dev)
        self.dgamma1, self.dbeta1 = self.small_grads[0:D], self.small_grads[D:2 * D]
        self.dgamma2, self.dbeta2 = self.small_grads[2 * D:3 * D], self.small_grads[3 * D:4 * D]
        self.dbias1 = self.small_grads[4 * D:]
        self.table_grad = torch.empty(V, D, device=dev)
        self.ws_ln = ops.ln_bwd_workspace(T, D, dev)
        self.ws_act = ops.act_bwd_workspace(capi.RELU, T, F, dev)
        self.ws_embed = ops.embed_workspace(T, V, D, dev)
        self.h_result = torch.empty(4 * D + F, dtype=torch.float32).pin_memory()
        self.readback = LaggedReadback(4 * D + F)
        self.side = torch.cuda.Stream()
        self.plan_ready = torch.cuda.Event()
        self.gather_done = torch.cuda.Event()
        self.plan_after_gather = plan_after_gather
        self.plan_on_main = False
        self.zero_done = torch.cuda.Event()
        if dist.active:
            Tg = T * dist.world
            self.Tg = Tg
            self.ids_all = torch.empty(Tg, dtype=torch.int32, device=dev)
            self.ws_global = ops.embed_workspace(Tg, V, D, dev)
            self.rank_plan = ops.embed_rank_plan_workspace(V, T, D, dev)
            self.h_used = torch.zeros(1, dtype=torch.int32).pin_memory()
            self.bwd_done, self.sums_done = torch.cuda.Event(), torch.cuda.Event()
            self.split_push = split_push
            # Table-gradient exchange: the library's fused scatter-add + peer-memory exchange, or (asked for, or when
            # symmetric memory cannot be set up) NCCL's all-reduce of the compacted rows.
            self.peer = None
            # Where the rows nobody uses are cleared: inside the push kernel (beside the NVLink-bound pushes),
            # or early on the second stream (beside the compute kernels).
            self.clear_early = clear == "early"
            self.clear_mode = {"early": 0, "fused": 1, "incremental": 2}[clear]
            self.exchange_note = "nccl all-reduce of the compacted rows"
            if exchange == "peer":
                try:
                    from dl_cuda_b200.sharding import PeerExchange
                    self.peer = PeerExchange(dist.dist, V, D, min(V, Tg), dev, tokens_per_rank=T,
                                             small_n=self.small_grads.numel())
                    # One barrier before anything depends on the flags; the verdict is shared, so either every
                    # rank uses the peer exchange or none does.
                    self.peer.barrier()
                    verdict = torch.tensor([self.peer.timed_out()], dtype=torch.int64, device=dev)
                    dist.dist.all_reduce(verdict, op=dist.dist.ReduceOp.MAX)
                    if int(verdict.item()) != 0:
                        raise RuntimeError("the peer barrier did not complete on every rank")
                    self.table_grad = self.peer.table_grad()
                    self.ids_all = self.peer.ids_all[:Tg]
                    self.exchange_note = ("scatter-add fused with a peer-memory exchange: rows one rank alone has tokens "
                                          "for go straight into every rank's dense table, shared rows to their owner, "
                                          "which adds them in rank order and stores the sum into every table")
                except Exception as exc:  # no symmetric memory on this box / build
                    self.peer = None
                    print(f"[bench] peer exchange unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
                    self.exchange_note += f" (peer exchange unavailable: {type(exc).__name__})"
            if self.peer is None:
                self.compact_rows = torch.empty(min(V, Tg), D, device=dev)
        self.distinct_ids = int(np.mean([np.unique(h.numpy()).size for h in self.h_id_sets]))

    # algorithmic HBM bytes of each op for the local tokens (each input byte read once,
    # each output byte written once)
    def bytes_per_op(self):
        T, D, F, V, S, e = self.T, self.D, self.F, self.V, self.S, self.e
        pos_rows = min(S, T)
        return {
            "sort_tokens": 0,
            "embed_gather_pe": (self.distinct_ids + T) * D * e + pos_rows * D * 4 + T * 4,
            "ln1_fwd": T * D * 4 * e + T * 4 + 2 * D * 4,
            "ln2_fwd": T * D * 4 * e + T * 4 + 2 * D * 4,
            "relu_fwd": T * F * 2 * e + T * F // 8 + F * 4,
            "relu_bwd": T * F * 2 * e + T * F // 8 + F * 4,
            "ln2_bwd": T * D * 3 * e + T * 4 + 3 * D * 4,
            "ln1_bwd": T * D * 4 * e + T * 4 + 3 * D * 4,
            # N > 1: only the rows used by some rank are written (the dense expansion is timed with the all-reduce)
            "embed_scatter": T * D * e + (self.used_rows() if self.dist.active else V) * D * 4 + T * 4,
            "allreduce": 0,
        }

    def used_rows(self) -> int:
        """Table rows some rank refers to, from the rank plan of the last step (synchronises)."""
        return int(self.rank_plan[:4].view(torch.int32)[0].item())

    def step(self, marks=None, copy_inputs=False, capture=None, lagged=False):
        lib, capi, st = self.lib, self.capi, torch.cuda.current_stream().cuda_stream
        p = lambda t: t.data_ptr()
        T, D, F, V, S, code = self.T, self.D, self.F, self.V, self.S, self.code
        chk = capi.check

        def mark():
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)

        self.h_ids, self.ids = self.h_id_sets[self.step_no % 2], self.id_sets[self.step_no % 2]
        self.step_no += 1
        if copy_inputs:
            self.ids.copy_(self.h_ids, non_blocking=True)
        mark()
        # The sorted-segment plan depends on the ids alone and is needed only by the last kernel of
        # backward: in the headline pass it is built on a side stream, beside the forward kernels.
        main = torch.cuda.current_stream()
        plan_stream = self.side if marks is None and not self.plan_on_main else main
        pst = plan_stream.cuda_stream
        if marks is None and not self.plan_on_main:
            self.side.wait_stream(main)
        plan_later = not self.dist.active and marks is None and self.plan_after_gather
        if plan_later:
            pass  # launched below, once the gather is in the queue
        elif not self.dist.active:
            chk(lib.dlb_embed_sort_tokens(p(self.ids), p(self.ws_embed), self.ws_embed.numel(), T, V, D, pst))
        else:
            # Every rank needs every rank's ids: one sort of the gathered list gives the numbering of the rows
            # used anywhere and each rank's tokens of them.  The gather is also the point where every rank is
            # known to be done with the previous step's tables.
            if self.peer is not None:
                self.peer.gather_ids(self.ids, stream=pst)
            else:
                with torch.cuda.stream(plan_stream):
                    self.dist.dist.all_gather_into_tensor(self.ids_all, self.ids)
            chk(lib.dlb_embed_sort_tokens(p(self.ids_all), p(self.ws_global), self.ws_global.numel(), self.Tg, V, D, pst))
            chk(lib.dlb_embed_rank_plan(p(self.ws_global), self.Tg, T, self.dist.world, self.dist.rank,
                                        p(self.rank_plan), self.rank_plan.numel(), V, D, pst))
            if self.peer is None:
                with torch.cuda.stream(plan_stream):
                    self.h_used.copy_(self.rank_plan[:4].view(torch.int32)[:1], non_blocking=True)
        if not plan_later:
            self.plan_ready.record(plan_stream)
        if self.dist.active and self.peer is not None and self.clear_early:
            # The rows nobody uses are cleared on the second stream as soon as the plan says which they are,
            # beside the forward and backward kernels (which, at a few thousand rows per GPU, leave HBM idle
            # between them).
            if plan_stream is not self.side:
                self.side.wait_event(self.plan_ready)
            chk(lib.dlb_embed_expand_rows(None, p(self.rank_plan), T, p(self.table_grad), V, D, 1, self.side.cuda_stream))
            self.zero_done.record(self.side)
        mark()
        chk(lib.dlb_embed_gather_fwd(p(self.table), p(self.ids), p(self.pe), S, p(self.x0), T, V, D, code, st))
        if plan_later:
            # One GPU: the plan (a latency-bound kernel of a few CTAs) starts once the gather has ended, beside
            # the first layer norm: next to the gather, whose CTAs each hold one position, it cost more.
            self.gather_done.record(main)
            self.side.wait_event(self.gather_done)
            chk(lib.dlb_embed_sort_tokens(p(self.ids), p(self.ws_embed), self.ws_embed.numel(), T, V, D, pst))
            self.plan_ready.record(plan_stream)
        mark()
        chk(lib.dlb_ln_residual_fwd(p(self.x0), p(self.attn_out), p(self.gamma1), p(self.beta1), p(self.y1),
                                    p(self.xhat1), p(self.inv1), T, D, 1e-5, code, st))
        mark()
        chk(lib.dlb_act_fwd(capi.RELU, p(self.ff_pre), p(self.bias1), p(self.act), p(self.mask), T, F, code, st))
        mark()
        chk(lib.dlb_ln_residual_fwd(p(self.y1), p(self.ff_out), p(self.gamma2), p(self.beta2), p(self.y2),
                                    p(self.xhat2), p(self.inv2), T, D, 1e-5, code, st))
        mark()
        chk(lib.dlb_ln_bwd(p(self.dy), None, p(self.xhat2), p(self.inv2), p(self.gamma2), p(self.dx2),
                           p(self.dgamma2), p(self.dbeta2), p(self.ws_ln), self.ws_ln.numel(), T, D, code, st))
        mark()
        chk(lib.dlb_act_bwd(capi.RELU, p(self.d_act), p(self.mask), p(self.d_pre), p(self.dbias1), p(self.ws_act),
                            self.ws_act.numel(), T, F, code, st))
        mark()
        chk(lib.dlb_ln_bwd(p(self.dx2), p(self.d_ff_in), p(self.xhat1), p(self.inv1), p(self.gamma1), p(self.dx1),
                           p(self.dgamma1), p(self.dbeta1), p(self.ws_ln), self.ws_ln.numel(), T, D, code, st))
        mark()
        if capture is not None:
            capture["small_local"] = self.small_grads.clone()
        if marks is None:
            main.wait_event(self.plan_ready)
        if not self.dist.active:
            chk(lib.dlb_embed_scatter_bwd(p(self.dx1), p(self.ids), p(self.table_grad), p(self.ws_embed),
                                          self.ws_embed.numel(), T, V, D, code, st))
            mark()
        elif self.peer is not None:
            px, ops = self.peer, self.ops
            # No host wait, no second stream and no library call between the kernels: the launches are sized
            # from upper bounds, the kernels read the exact row counts, zero the rows nobody uses, announce their
            # stores and wait for the other ranks themselves.
            pushed, done = px.next_epoch(px.CH_PUSHED), px.next_epoch(px.CH_DONE)
            scatter = lambda part, stream: ops.embed_scatter_bwd_peer(
                self.dx1, self.ws_global, self.Tg, self.rank_plan, T, px.group, self.small_grads, min(V, self.Tg), V,
                px.CH_PUSHED, pushed, clear_unused=self.clear_mode, part=part, stream=stream)
            if marks is None and self.split_push:
                # The rows with one token need no sum: they go out (with the clearing) while the second stream
                # adds up the rows with several tokens; those follow, and with them the announcement.
                self.bwd_done.record(main)
                self.side.wait_event(self.bwd_done)
                scatter(1, self.side.cuda_stream)
                self.sums_done.record(self.side)
                scatter(2, st)
                main.wait_event(self.sums_done)
                scatter(3, st)
            else:
                scatter(0, st)
            mark()
            ops.embed_reduce_broadcast_peer(self.rank_plan, T, px.group, self.small_grads, V, D, code, px.CH_PUSHED,
                                            pushed, px.CH_DONE, done, stream=st)
            if self.clear_early:
                main.wait_event(self.zero_done)
            px.wait(px.CH_DONE, stream=st)  # every rank's table holds every row
        else:
            # Compacted form through NCCL: only the rows some rank uses are summed, all-reduced and expanded.
            self.plan_ready.synchronize()  # the row count is a host argument of the all-reduce
            used = int(self.h_used[0])
            chk(lib.dlb_embed_scatter_bwd_compact(p(self.dx1), p(self.ws_global), self.Tg, p(self.rank_plan), T,
                                                  self.dist.rank, p(self.compact_rows), used, V, D, code, st))
            mark()
            # zero the unused rows of the dense gradient beside the all-reduce
            self.side.wait_stream(main)
            chk(lib.dlb_embed_expand_rows(None, p(self.rank_plan), T, p(self.table_grad), V, D, 1, self.side.cuda_stream))
            self.zero_done.record(self.side)
            allreduce_param_grads(self.dist.dist, self.small_grads, self.compact_rows[:used])
            main.wait_event(self.zero_done)
            chk(lib.dlb_embed_expand_rows(p(self.compact_rows), p(self.rank_plan), T, p(self.table_grad), V, D, 2, st))
        mark()
        if copy_inputs and lagged:
            return self.readback.push(self.small_grads)
        if copy_inputs:
            self.h_result.copy_(self.small_grads, non_blocking=True)
            main.synchronize()
            return float(self.h_result[0])
        return None

    # ---- the exchange of step i beside the forward pass of step i+1 (an extra figure, not the headline) ----
    def enable_overlap(self):
        """A second set of everything the exchange touches (peer buffers with their own dense table, global plan,
        rank plan, reduced small gradients) and a stream of its own for the exchange kernels, so that step i+1
        can start while the table gradient of step i is still on its way.  Returns False where the peer
        exchange is not in use."""
        if self.peer is None:
            return False
        from dl_cuda_b200.sharding import PeerExchange
        ops, dev, T, D, V = self.ops, self.table.device, self.T, self.D, self.V
        second = PeerExchange(self.dist.dist, V, D, min(V, self.Tg), dev, tokens_per_rank=T,
                              small_n=self.small_grads.numel())
        second.barrier()
        verdict = torch.tensor([second.timed_out()], dtype=torch.int64, device=dev)
        self.dist.dist.all_reduce(verdict, op=self.dist.dist.ReduceOp.MAX)
        if int(verdict.item()) != 0:
            return False
        mk = lambda peer, ws_global, rank_plan: dict(
            peer=peer, ws_global=ws_global, rank_plan=rank_plan, table_grad=peer.table_grad(),
            small_out=torch.empty_like(self.small_grads), plan_ready=torch.cuda.Event(), done=torch.cuda.Event())
        self.sets = [mk(self.peer, self.ws_global, self.rank_plan),
                     mk(second, ops.embed_workspace(self.Tg, V, D, dev), ops.embed_rank_plan_workspace(V, T, D, dev))]
        self.ex = torch.cuda.Stream(priority=-1)
        self.ex_pushed = torch.cuda.Event()
        self.ov_step = 0
        return True

    def step_overlapped(self):
        """One step whose table-gradient exchange runs on its own stream: the next step's kernels do not wait for
        it.  Step i uses buffer set i % 2; a set is reused once ITS last exchange has ended on this rank, and
        the gather of the token ids that opens a step is where the ranks learn that of one another."""
        lib, capi, ops = self.lib, self.capi, self.ops
        p = lambda t: t.data_ptr()
        T, D, F, V, S, code = self.T, self.D, self.F, self.V, self.S, self.code
        chk = capi.check
        main, side, ex = torch.cuda.current_stream(), self.side, self.ex
        st, sst = main.cuda_stream, side.cuda_stream
        cur = self.sets[self.ov_step % 2]
        ids = self.id_sets[self.ov_step % 2]
        self.ids = ids
        self.ov_step += 1
        px = cur["peer"]
        # plan of this step on the second stream, in this set's buffers
        side.wait_event(cur["done"])
        px.gather_ids(ids, stream=sst)
        chk(lib.dlb_embed_sort_tokens(p(px.ids_all), p(cur["ws_global"]), cur["ws_global"].numel(), self.Tg, V, D, sst))
        chk(lib.dlb_embed_rank_plan(p(cur["ws_global"]), self.Tg, T, self.dist.world, self.dist.rank,
                                    p(cur["rank_plan"]), cur["rank_plan"].numel(), V, D, sst))
        cur["plan_ready"].record(side)
        # forward
        chk(lib.dlb_embed_gather_fwd(p(self.table), p(ids), p(self.pe), S, p(self.x0), T, V, D, code, st))
        chk(lib.dlb_ln_residual_fwd(p(self.x0), p(self.attn_out), p(self.gamma1), p(self.beta1), p(self.y1),
                                    p(self.xhat1), p(self.inv1), T, D, 1e-5, code, st))
        chk(lib.dlb_act_fwd(capi.RELU, p(self.ff_pre), p(self.bias1), p(self.act), p(self.mask), T, F, code, st))
        chk(lib.dlb_ln_residual_fwd(p(self.y1), p(self.ff_out), p(self.gamma2), p(self.beta2), p(self.y2),
                                    p(self.xhat2), p(self.inv2), T, D, 1e-5, code, st))
        # backward writes the small gradients and dx1, which the exchange of the step before still may read
        main.wait_event(self.ex_pushed)
        chk(lib.dlb_ln_bwd(p(self.dy), None, p(self.xhat2), p(self.inv2), p(self.gamma2), p(self.dx2),
                           p(self.dgamma2), p(self.dbeta2), p(self.ws_ln), self.ws_ln.numel(), T, D, code, st))
        chk(lib.dlb_act_bwd(capi.RELU, p(self.d_act), p(self.mask), p(self.d_pre), p(self.dbias1), p(self.ws_act),
                            self.ws_act.numel(), T, F, code, st))
        chk(lib.dlb_ln_bwd(p(self.dx2), p(self.d_ff_in), p(self.xhat1), p(self.inv1), p(self.gamma1), p(self.dx1),
                           p(self.dgamma1), p(self.dbeta1), p(self.ws_ln), self.ws_ln.numel(), T, D, code, st))
        self.bwd_done.record(main)
        # the exchange, on its own stream
        ex.wait_event(self.bwd_done)
        ex.wait_event(cur["plan_ready"])
        xst = ex.cuda_stream
        pushed, done = px.next_epoch(px.CH_PUSHED), px.next_epoch(px.CH_DONE)
        ops.embed_scatter_bwd_peer(self.dx1, cur["ws_global"], self.Tg, cur["rank_plan"], T, px.group, self.small_grads,
                                   min(V, self.Tg), V, px.CH_PUSHED, pushed, clear_unused=self.clear_mode, part=0, stream=xst)
        self.ex_pushed.record(ex)
        ops.embed_reduce_broadcast_peer(cur["rank_plan"], T, px.group, cur["small_out"], V, D, code, px.CH_PUSHED,
                                        pushed, px.CH_DONE, done, stream=xst)
        px.wait(px.CH_DONE, stream=xst)
        cur["done"].record(ex)
        return cur

    def drain_overlapped(self):
        """The main stream waits for the exchange still in flight (the end of a timed region)."""
        torch.cuda.current_stream().wait_stream(self.ex)

    def verify_overlapped(self):
        """Untimed: overlapped steps, then the table and the small gradients of the LAST step (whose inputs are
        still in place) against the single-rank result of all tokens; once for each buffer set."""
        d, ops = self.dist.dist, self.ops
        T, D, V, Tg = self.T, self.D, self.V, self.Tg
        worst_table = worst_small = 0.0
        for steps in (3, 1):  # the last step lands in set 0, then in set 1
            for _ in range(steps):
                cur = self.step_overlapped()
            self.drain_overlapped()
            torch.cuda.synchronize()
            dx_all = torch.empty(Tg, D, dtype=self.dtype, device=self.dx1.device)
            d.all_gather_into_tensor(dx_all, self.dx1)
            ids_all = torch.empty(Tg, dtype=torch.int32, device=self.dx1.device)
            d.all_gather_into_tensor(ids_all, self.ids)
            want = ops.embed_scatter_bwd(dx_all, ids_all, V, ops.embed_sort_tokens(ids_all, V, D))
            worst_table = max(worst_table, rel_err_rows_dev(cur["table_grad"], want))
            del want, dx_all
            small_all = torch.empty(self.dist.world, self.small_grads.numel(), device=self.dx1.device)
            d.all_gather_into_tensor(small_all, self.small_grads)
            worst_small = max(worst_small, rel_err_dev(cur["small_out"], small_all.double().sum(0)))
        status = 0
        for cur in self.sets:
            status |= cur["peer"].timed_out()
        worst = torch.tensor([worst_table, worst_small, float(status != 0)], dtype=torch.float64, device=self.dx1.device)
        d.all_reduce(worst, op=d.ReduceOp.MAX)
        return {"max_rel_err_table_grad": float(worst[0]), "max_rel_err_small_grads": float(worst[1]),
                "status_bits_clear": float(worst[2]) == 0.0, "tolerance": 1e-5}

    def verify(self):
        """N > 1, untimed: one step, then every rank checks its dense table gradient and its reduced small
        gradients against the single-rank result of ALL tokens (the other ranks' gradients and ids are
        gathered here only for the check), and that every rank holds the same bits as rank 0."""
        d, ops, lib = self.dist.dist, self.ops, self.lib
        captured = {}
        self.step(capture=captured)
        torch.cuda.synchronize()
        T, D, V, Tg = self.T, self.D, self.V, self.Tg
        dx_all = torch.empty(Tg, D, dtype=self.dtype, device=self.dx1.device)
        d.all_gather_into_tensor(dx_all, self.dx1)
        ids_all = torch.empty(Tg, dtype=torch.int32, device=self.dx1.device)
        d.all_gather_into_tensor(ids_all, self.ids)
        plan = ops.embed_sort_tokens(ids_all, V, D)
        want = ops.embed_scatter_bwd(dx_all, ids_all, V, plan)
        err_table = rel_err_rows_dev(self.table_grad, want)
        err_table_rms = rel_err_dev(self.table_grad, want)
        del want, dx_all
        small_all = torch.empty(self.dist.world, self.small_grads.numel(), device=self.dx1.device)
        d.all_gather_into_tensor(small_all, captured["small_local"])
        err_small = rel_err_dev(self.small_grads, small_all.double().sum(0))
        mine = torch.cat([self.table_grad.reshape(-1), self.small_grads])
        theirs = mine.clone()
        d.broadcast(theirs, src=0)
        same = torch.tensor([1 if same_bits(mine, theirs) else 0], dtype=torch.int32, device=mine.device)
        d.all_reduce(same, op=d.ReduceOp.MIN)
        worst = torch.tensor([err_table, err_small, err_table_rms], dtype=torch.float64, device=mine.device)
        d.all_reduce(worst, op=d.ReduceOp.MAX)
        gave_up = self.peer.timed_out() if self.peer is not None else 0
        return {"max_rel_err_table_grad": float(worst[0]), "max_rel_err_small_grads": float(worst[1]),
                "max_rel_err_table_grad_vs_table_rms": float(worst[2]),
                "ranks_bit_identical": bool(int(same.item())), "status_bits": gave_up,
                "against": "the single-rank gradient of all tokens (same kernels, one GPU's association)",
                "measure": "|a-b| / max(|a|, |b|, rms of the element's own table row); small gradients: rms of the vector",
                "tolerance": 1e-5}


# --------------------------------------------------------------------------- the chain (reference kernels)
class ReferenceChain:
    """The same chain through the reference's own CUDA kernels (fp32 only, default stream)."""

    def __init__(self, tokens, seq, d, f, vocab, seed, inputs=None):
        from oracle import ref
        self.ref = ref
        dev = torch.device("cuda", torch.cuda.current_device())
        T, D, F, V = tokens, d, f, vocab
        self.T, self.S, self.D, self.F, self.V = T, seq, D, F, V
        self.bias1 = None  # the timed arm adds no bias: the reference does that inside its GEMM kernel
        if inputs is None:
            g = torch.Generator(device=dev)
            g.manual_seed(seed)
            randn = lambda *s: torch.randn(*s, generator=g, device=dev)
            self.table = randn(V, D) * 0.02
            self.pe = ref.pe_table(seq, D).to(dev)
            self.gamma1 = self.gamma2 = torch.rand(D, generator=g, device=dev) + 0.5
            self.beta1 = self.beta2 = randn(D) * 0.1
            rng = np.random.Generator(np.random.Philox(key=seed))
            self.h_ids = torch.from_numpy(zipf_ids(rng, T, V)).pin_memory()
            self.ids = self.h_ids.to(dev)
            self.attn_out, self.ff_out, self.dy, self.d_ff_in = randn(T, D), randn(T, D), randn(T, D), randn(T, D)
            self.ff_pre, self.d_act = randn(T, F), randn(T, F)
        else:
            for name, value in inputs.items():
                setattr(self, name, value)
        e = lambda *s: torch.empty(*s, device=dev)
        self.emb, self.x0, self.res, self.y1, self.xhat1, self.y2, self.xhat2 = (e(T, D) for _ in range(7))
        self.inv1, self.inv2 = e(T), e(T)
        self.act, self.relu_cache, self.d_pre = e(T, F), e(T, F), e(T, F)
        self.dx2, self.dsum, self.dx1, self.dpe = e(T, D), e(T, D), e(T, D), e(T, D)
        self.small = e(4 * D + F)
        self.table_grad = e(V, D)
        self.h_result = torch.empty(4 * D + F).pin_memory()

    @classmethod
    def from_inputs(cls, chain: "Chain"):
        """The reference chain on the inputs of a native chain (storage widened to fp32), with the FFN
        bias added in a pass of its own: for comparing results, not for timing."""
        f = lambda t: t.float()
        inputs = dict(table=f(chain.table), pe=chain.pe, gamma1=chain.gamma1, beta1=chain.beta1,
                      gamma2=chain.gamma2, beta2=chain.beta2, h_ids=chain.h_ids, ids=chain.ids,
                      attn_out=f(chain.attn_out), ff_out=f(chain.ff_out), dy=f(chain.dy),
                      d_ff_in=f(chain.d_ff_in), ff_pre=f(chain.ff_pre), d_act=f(chain.d_act))
        self = cls(chain.T, chain.S, chain.D, chain.F, chain.V, seed=0, inputs=inputs)
        self.bias1 = chain.bias1
        self.pre = torch.empty_like(self.ff_pre)
        return self

    def step(self, copy_inputs=False, lagged=False):
        r, D, F = self.ref, self.D, self.F
        B = self.T // self.S if self.T >= self.S else 1
        S = min(self.S, self.T)
        if copy_inputs:
            self.ids.copy_(self.h_ids, non_blocking=True)
        r.lib().ref_embed_fwd(self.table.data_ptr(), self.ids.data_ptr(), self.emb.data_ptr(), self.T, D)
        r.lib().ref_pe_add(self.emb.data_ptr(), self.pe.data_ptr(), self.x0.data_ptr(), B, S, D)
        n = self.T * D
        r.lib().ref_residual_add(self.x0.data_ptr(), self.attn_out.data_ptr(), self.res.data_ptr(), n)
        r.lib().ref_ln_fwd(self.res.data_ptr(), self.gamma1.data_ptr(), self.beta1.data_ptr(), self.y1.data_ptr(),
                           self.xhat1.data_ptr(), self.inv1.data_ptr(), self.T, D, 1e-5)
        # the bias add of the reference is the last line of its GEMM kernel: nothing extra to time
        pre = self.ff_pre
        if self.bias1 is not None:
            r.lib().ref_bias_add(self.ff_pre.data_ptr(), self.bias1.data_ptr(), self.pre.data_ptr(), self.T, F)
            pre = self.pre
        r.lib().ref_act_fwd(0, pre.data_ptr(), self.act.data_ptr(), self.relu_cache.data_ptr(), self.T * F)
        r.lib().ref_residual_add(self.y1.data_ptr(), self.ff_out.data_ptr(), self.res.data_ptr(), n)
        r.lib().ref_ln_fwd(self.res.data_ptr(), self.gamma2.data_ptr(), self.beta2.data_ptr(), self.y2.data_ptr(),
                           self.xhat2.data_ptr(), self.inv2.data_ptr(), self.T, D, 1e-5)
        s = self.small
        r.lib().ref_ln_bwd(self.dy.data_ptr(), self.xhat2.data_ptr(), self.inv2.data_ptr(), self.gamma2.data_ptr(),
                           self.dx2.data_ptr(), s[2 * D:].data_ptr(), s[3 * D:].data_ptr(), self.T, D)
        r.lib().ref_act_bwd(0, self.d_act.data_ptr(), self.relu_cache.data_ptr(), self.d_pre.data_ptr(), self.T * F)
        r.lib().ref_bias_grad(self.d_pre.data_ptr(), s[4 * D:].data_ptr(), self.T, F)
        r.lib().ref_residual_add(self.dx2.data_ptr(), self.d_ff_in.data_ptr(), self.dsum.data_ptr(), n)
        r.lib().ref_ln_bwd(self.dsum.data_ptr(), self.xhat1.data_ptr(), self.inv1.data_ptr(), self.gamma1.data_ptr(),
                           self.dx1.data_ptr(), s[0:].data_ptr(), s[D:].data_ptr(), self.T, D)
        r.lib().ref_pe_bwd(self.dx1.data_ptr(), self.dpe.data_ptr(), n)
        code = r.lib().ref_embed_bwd(self.dpe.data_ptr(), self.ids.data_ptr(), self.table_grad.data_ptr(), self.T,
                                     self.V, D)
        if code != 0:
            raise RuntimeError(f"reference kernels failed: CUDA error {code}")
        if copy_inputs and lagged:
            if not hasattr(self, "readback"):
                self.readback = LaggedReadback(self.small.numel())
            return self.readback.push(self.small)
        if copy_inputs:
            self.h_result.copy_(self.small, non_blocking=True)
            torch.cuda.synchronize()
            return float(self.h_result[0])
        return None


# --------------------------------------------------------------------------- host baseline
def cpu_baseline(sample_tokens=16384):
    """The chain through the single-threaded host loops of oracle/host_ref.cpp on a slice of
    the tokens (fp32 host arrays; the table gradient is produced at full vocabulary size)."""
    from oracle import cpu
    lib = cpu.lib()
    T, D, F, V, S = sample_tokens, D_MODEL, D_FF, VOCAB, SEQ
    rng = np.random.Generator(np.random.Philox(key=9))
    f32 = lambda *s: rng.standard_normal(s, dtype=np.float32)
    table, pe = f32(V, D) * np.float32(0.02), cpu.pe_table(S, D)
    ids = zipf_ids(rng, T, V)
    attn, ffo, dy, dffi = f32(T, D), f32(T, D), f32(T, D), f32(T, D)
    ffpre, dact = f32(T, F), f32(T, F)
    gamma, beta, bias = np.ones(D, np.float32), np.zeros(D, np.float32), np.zeros(F, np.float32)
    z = lambda *s: np.zeros(s, np.float32)  # zeros: pages are touched before the clock starts
    x0, y1, xh1, y2, xh2, dx2, dx1 = (z(T, D) for _ in range(7))
    inv1, inv2 = z(T), z(T)
    act, pre, dpre = z(T, F), z(T, F), z(T, F)
    dg, db, dbias, grad = z(D), z(D), z(F), z(V, D)
    P = lambda a: ctypes.c_void_p(a.ctypes.data)
    i64 = ctypes.c_int64
    t0 = time.perf_counter()
    lib.orc_embed_gather(P(table), P(ids), P(pe), S, P(x0), T, D)
    lib.orc_ln_residual_fwd(P(x0), P(attn), P(gamma), P(beta), P(y1), P(xh1), P(inv1), T, D, ctypes.c_float(1e-5))
    lib.orc_act_fwd(0, P(ffpre), P(bias), P(act), P(pre), i64(T), i64(F))
    lib.orc_ln_residual_fwd(P(y1), P(ffo), P(gamma), P(beta), P(y2), P(xh2), P(inv2), T, D, ctypes.c_float(1e-5))
    lib.orc_ln_bwd_dx(P(dy), None, P(xh2), P(inv2), P(gamma), P(dx2), T, D)
    lib.orc_ln_param_grad(P(dy), None, P(xh2), P(dg), P(db), T, D)
    lib.orc_act_bwd(0, P(dact), P(pre), P(dpre), i64(T * F))
    lib.orc_bias_grad(P(dpre), P(dbias), i64(T), i64(F))
    lib.orc_ln_bwd_dx(P(dx2), P(dffi), P(xh1), P(inv1), P(gamma), P(dx1), T, D)
    lib.orc_ln_param_grad(P(dx2), P(dffi), P(xh1), P(dg), P(db), T, D)
    lib.orc_embed_scatter(P(dx1), P(ids), P(grad), T, V, D)
    dt = time.perf_counter() - t0
    return {"value": T / dt, "unit": "tokens/s", "cores": 1, "kind": "port",
            "host_cores_available": os.cpu_count(),
            "sample": f"{T} of {BATCH * SEQ} tokens through the whole fp32 chain in {dt:.1f} s, "
                      f"single thread, table gradient at full vocab {V}x{D}"}


# --------------------------------------------------------------------------- per-kernel sweep (fp32 large configs)
def time_op(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    evs[0].record()
    for i in range(iters):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    return float(np.mean([evs[i].elapsed_time(evs[i + 1]) for i in range(iters)]))


def rel_err_dev(got, want) -> float:
    """max |got-want| / max(|got|, |want|, rms(want)) evaluated on the device in fp64, in slices."""
    got, want = got.reshape(-1), want.reshape(-1)
    n, step = want.numel(), 1 << 26
    sq = 0.0
    for i in range(0, n, step):
        w = want[i:i + step].double()
        sq += float((w * w).sum())
    rms = max((sq / max(n, 1)) ** 0.5, 1e-30)
    worst = 0.0
    for i in range(0, n, step):
        g, w = got[i:i + step].double(), want[i:i + step].double()
        denom = torch.maximum(torch.maximum(g.abs(), w.abs()), torch.full_like(w, rms))
        worst = max(worst, float(((g - w).abs() / denom).max()))
    return worst


def rel_err_rows_dev(got, want) -> float:
    """rel_err_dev with the rms of each ROW of `want` as the floor of the denominator: a table gradient is
    mostly zero rows beside a few rows that sum thousands of terms, so the rms of the whole tensor says
    nothing about the scale of either kind (a hot row's fp32 sum is then "off" by 1e-5 of that rms whatever
    the order of its additions).  A zero row must be matched exactly."""
    worst = 0.0
    for r0 in range(0, want.shape[0], 4096):
        g, w = got[r0:r0 + 4096].double(), want[r0:r0 + 4096].double()
        rms = (w * w).mean(dim=1, keepdim=True).sqrt()
        denom = torch.maximum(torch.maximum(g.abs(), w.abs()), rms).clamp_min(1e-300)
        worst = max(worst, float(((g - w).abs() / denom).max()))
    return worst


def same_bits(a, b) -> bool:
    return a.shape == b.shape and bool(torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32)))


def kernel_sweep(peak, with_reference=False):
    """GB/s of each kernel on the large fp32 configurations (inputs far larger than L2).  With
    `with_reference` (a baseline leg: it runs the shim around the reference's own kernels) every
    entry of configs 2-4 also carries the time of the reference's kernels for the same op on the
    same inputs, the speed-up, and the largest relative error between the two results."""
    from dl_cuda_b200 import capi, ops
    ref = None
    if with_reference:
        from oracle import ref as ref_mod
        ref = ref_mod if ref_mod.available() else None
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    randn = lambda *s: torch.randn(*s, generator=g, device=dev)
    out = []

    def add(name, cfg, nbytes, ms, ref_fn=None, compare=None, exact=None):
        gbs = nbytes / ms / 1e6
        entry = {"kernel": name, "config": cfg, "ms": round(ms, 4), "bytes": int(nbytes),
                 "gbs": round(gbs, 1), "frac_measured": round(gbs / peak, 4),
                 "frac_nominal": round(gbs / NOMINAL_HBM_GBS, 4)}
        if ref is not None and ref_fn is not None:
            ref_ms = time_op(ref_fn, warmup=1, iters=3)
            entry["ref_ms"] = round(ref_ms, 4)
            entry["speedup_vs_ref"] = round(ref_ms / ms, 2)
            if compare is not None:
                errs = compare()
                entry["max_rel_err_vs_ref"] = max(errs.values())
                entry["err_vs_ref"] = {k: float(f"{v:.3g}") for k, v in errs.items()}
                entry["bit_exact_vs_ref"] = all(v == 0.0 for v in errs.values())
            if exact is not None:
                # reductions: this library and the reference each against the sum in fp64 (the reference adds
                # its terms one by one in fp32, so its own distance from the exact sum bounds any agreement)
                mine, theirs = exact()
                entry["err_vs_fp64"] = {k: float(f"{v:.3g}") for k, v in mine.items()}
                entry["ref_err_vs_fp64"] = {k: float(f"{v:.3g}") for k, v in theirs.items()}
        out.append(entry)

    bits = lambda a, b: 0.0 if same_bits(a, b) else max(rel_err_dev(a, b), 1e-30)

    def colsum64(*factors):
        """Column sums of the element-wise product of 2-D tensors, accumulated in fp64 in row slices."""
        acc = torch.zeros(factors[0].shape[1], dtype=torch.float64, device=dev)
        for r0 in range(0, factors[0].shape[0], 4096):
            prod = factors[0][r0:r0 + 4096].double()
            for f in factors[1:]:
                prod = prod * f[r0:r0 + 4096].double()
            acc += prod.sum(0)
        return acc

    def ln_exact(dy_a, dy_b):
        def run():
            dsum = dy_a if dy_b is None else dy_a + dy_b  # one rounding, as both implementations do
            g64, b64 = colsum64(dsum, xhat), colsum64(dsum)
            return ({"dgamma": rel_err_dev(dg, g64), "dbeta": rel_err_dev(db, b64)},
                    {"dgamma": rel_err_dev(dg_r, g64), "dbeta": rel_err_dev(db_r, b64)})
        return run

    # config 1: char-LM shapes (batch 32 x seq 64, d_model 64, vocab 65, FFN 2048 x 256): launch-latency
    # bound (every tensor fits L2), so the time per call is what matters; GB/s only for information
    T1, D1, V1, S1, F1 = 2048, 64, 65, 64, 256
    a1, b1, dy1 = randn(T1, D1), randn(T1, D1), randn(T1, D1)
    g1, be1 = torch.ones(D1, device=dev), torch.zeros(D1, device=dev)
    y1, xh1, inv1 = torch.empty_like(a1), torch.empty_like(a1), torch.empty(T1, device=dev)
    dx1, dg1, db1 = torch.empty_like(a1), torch.empty(D1, device=dev), torch.empty(D1, device=dev)
    ws1 = ops.ln_bwd_workspace(T1, D1, dev)
    tab1 = randn(V1, D1) * 0.02
    ids1 = torch.randint(0, V1, (T1,), generator=g, device=dev, dtype=torch.int32)
    pe1, out1, grad1 = ops.pe_table(S1, D1).to(dev), torch.empty(T1, D1, device=dev), torch.empty(V1, D1, device=dev)
    wse1 = ops.embed_workspace(T1, V1, D1, dev)
    x1, dyf1, bias1 = randn(T1, F1), randn(T1, F1), randn(F1) * 0.1
    yf1, dxf1, dbias1 = torch.empty_like(x1), torch.empty_like(x1), torch.empty(F1, device=dev)
    wsa1 = ops.act_bwd_workspace(capi.RELU, T1, F1, dev)
    cfg1 = "char-LM shapes 2048x64 / V65 / 2048x256 fp32"
    it = dict(iters=50)
    add("residual_add", cfg1, T1 * D1 * 12, time_op(lambda: ops.residual_add(a1, b1, out=y1), **it))
    add("ln_residual_fwd", cfg1, T1 * D1 * 16, time_op(lambda: ops.ln_residual_fwd(a1, b1, g1, be1, 1e-5, y=y1, xhat=xh1, inv_std=inv1), **it))
    add("ln_bwd", cfg1, T1 * D1 * 12, time_op(lambda: ops.ln_bwd(dy1, None, xh1, inv1, g1, dx=dx1, dgamma=dg1, dbeta=db1, workspace=ws1), **it))
    add("ln_bwd_two_grads", cfg1, T1 * D1 * 16, time_op(lambda: ops.ln_bwd(dy1, b1, xh1, inv1, g1, dx=dx1, dgamma=dg1, dbeta=db1, workspace=ws1), **it))
    add("embed_gather_pe_fwd", cfg1, T1 * D1 * 8, time_op(lambda: ops.embed_gather_fwd(tab1, ids1, pe1, S1, out=out1), **it))
    add("embed_gather_fwd", cfg1, T1 * D1 * 8, time_op(lambda: ops.embed_gather_fwd(tab1, ids1, None, 0, out=out1), **it))
    add("pe_add_fwd", cfg1, T1 * D1 * 8, time_op(lambda: ops.pe_add_fwd(a1.view(T1 // S1, S1, D1), pe1, out=y1.view(T1 // S1, S1, D1)), **it))
    add("pe_add_bwd", cfg1, T1 * D1 * 8, time_op(lambda: ops.pe_add_bwd(dy1, dx=dx1), **it))
    add("embed_sort_tokens", cfg1, 0, time_op(lambda: ops.embed_sort_tokens(ids1, V1, D1, workspace=wse1), **it))
    add("embed_scatter_bwd", cfg1, T1 * D1 * 4 + V1 * D1 * 4, time_op(lambda: ops.embed_scatter_bwd(dy1, ids1, V1, wse1, grad=grad1), **it))
    for kind, name in ((capi.RELU, "relu"), (capi.SIGMOID, "sigmoid"), (capi.TANH, "tanh")):
        c1 = ops.act_cache(kind, x1)
        cache_b = T1 * F1 // 8 if kind == capi.RELU else T1 * F1 * 4
        add(f"bias_{name}_fwd", cfg1, T1 * F1 * 8 + cache_b, time_op(lambda: ops.act_fwd(kind, x1, bias1, y=yf1, cache=c1), **it))
        add(f"{name}_bwd", cfg1, T1 * F1 * 8 + cache_b, time_op(lambda: ops.act_bwd(kind, dyf1, c1, dx=dxf1), **it))
        add(f"{name}_bwd_dbias", cfg1, T1 * F1 * 8 + cache_b, time_op(lambda: ops.act_bwd(kind, dyf1, c1, dx=dxf1, dbias=dbias1, want_dbias=True, workspace=wsa1), **it))
    wsb1 = torch.empty(max(capi.lib().dlb_bias_grad_workspace_bytes(T1, F1), 16), dtype=torch.uint8, device=dev)
    add("bias_grad", cfg1, T1 * F1 * 4, time_op(lambda: ops.bias_grad(dyf1, dbias=dbias1, workspace=wsb1), **it))
    c1 = ops.act_cache(capi.RELU, x1)

    # The same seven calls as ONE CUDA graph: at these sizes the host's per-call cost dominates the figures
    # above, a replayed graph shows what the GPU itself needs for the whole forward + backward chain.
    def chain1():
        ops.embed_sort_tokens(ids1, V1, D1, workspace=wse1)
        ops.embed_gather_fwd(tab1, ids1, pe1, S1, out=out1)
        ops.ln_residual_fwd(out1, b1, g1, be1, 1e-5, y=y1, xhat=xh1, inv_std=inv1)
        ops.act_fwd(capi.RELU, x1, None, y=yf1, cache=c1)
        ops.act_bwd(capi.RELU, dyf1, c1, dx=dxf1)
        ops.ln_bwd(dy1, None, xh1, inv1, g1, dx=dx1, dgamma=dg1, dbeta=db1, workspace=ws1)
        ops.embed_scatter_bwd(dx1, ids1, V1, wse1, grad=grad1)

    chain_bytes = T1 * D1 * (16 + 12 + 8 + 4) + V1 * D1 * 4 + 2 * T1 * F1 * 8
    try:
        eager_ms = time_op(chain1, iters=50)
        want = None
        chain1()
        want = grad1.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            chain1()
        grad1.zero_()
        graph.replay()
        torch.cuda.synchronize()
        if not torch.equal(grad1, want):
            raise RuntimeError("graph replay differs from the eager chain")
        add("chain_eager_7_calls", cfg1, chain_bytes, eager_ms)
        add("chain_cuda_graph_replay", cfg1, chain_bytes, time_op(graph.replay, iters=50))
    except Exception as exc:  # a capture problem must not cost the benchmark its headline
        print(f"[bench] CUDA graph of the char-LM chain skipped: {type(exc).__name__}: {exc}", file=sys.stderr)

    # config 2: LN + residual, 65536 x 1024
    R, D = 65536, 1024
    a, b, dy = randn(R, D), randn(R, D), randn(R, D)
    gamma, beta = torch.rand(D, generator=g, device=dev) + 0.5, randn(D) * 0.1
    y, xhat, inv = torch.empty_like(a), torch.empty_like(a), torch.empty(R, device=dev)
    dx, dg, db = torch.empty_like(a), torch.empty(D, device=dev), torch.empty(D, device=dev)
    ws = ops.ln_bwd_workspace(R, D, dev)
    if ref is not None:
        s_r, y_r, xhat_r, inv_r = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a), torch.empty(R, device=dev)
        dx_r, dg_r, db_r = torch.empty_like(a), torch.empty(D, device=dev), torch.empty(D, device=dev)
    cfg2 = "65536x1024 fp32"
    ms = time_op(lambda: ops.ln_residual_fwd(a, b, gamma, beta, 1e-5, y=y, xhat=xhat, inv_std=inv))
    add("ln_residual_fwd", cfg2, R * D * 16 + R * 4 + 2 * D * 4, ms,
        lambda: ref.ln_fwd(ref.residual_add(a, b, out=s_r), gamma, beta, 1e-5, y=y_r, xhat=xhat_r, inv_std=inv_r),
        lambda: {"y": rel_err_dev(y, y_r), "xhat": rel_err_dev(xhat, xhat_r), "inv_std": rel_err_dev(inv, inv_r)})
    ms = time_op(lambda: ops.ln_bwd(dy, None, xhat, inv, gamma, dx=dx, dgamma=dg, dbeta=db, workspace=ws))
    add("ln_bwd", cfg2, R * D * 12 + R * 4 + 3 * D * 4, ms,
        lambda: ref.ln_bwd(dy, xhat, inv, gamma, dx=dx_r, dgamma=dg_r, dbeta=db_r),
        lambda: {"dx": rel_err_dev(dx, dx_r), "dgamma": rel_err_dev(dg, dg_r), "dbeta": rel_err_dev(db, db_r)},
        ln_exact(dy, None))
    ms = time_op(lambda: ops.ln_bwd(dy, b, xhat, inv, gamma, dx=dx, dgamma=dg, dbeta=db, workspace=ws))
    add("ln_bwd_two_grads", cfg2, R * D * 16 + R * 4 + 3 * D * 4, ms,
        lambda: ref.ln_bwd(ref.residual_add(dy, b, out=s_r), xhat, inv, gamma, dx=dx_r, dgamma=dg_r, dbeta=db_r),
        lambda: {"dx": rel_err_dev(dx, dx_r), "dgamma": rel_err_dev(dg, dg_r), "dbeta": rel_err_dev(db, db_r)},
        ln_exact(dy, b))
    del a, b, dy, y, xhat, dx
    if ref is not None:
        del s_r, y_r, xhat_r, dx_r

    # config 3: embedding + PE, vocab 32000 x 4096, 16 x 2048 Zipf tokens
    V, D, B, S = 32000, 4096, 16, 2048
    T = B * S
    table = randn(V, D) * 0.02
    ids_h = zipf_ids(np.random.Generator(np.random.Philox(key=1236)), T, V)
    ids = torch.from_numpy(ids_h).to(dev)
    U = int(np.unique(ids_h).size)
    pe = ops.pe_table(S, D).to(dev)
    outb, dyb = torch.empty(T, D, device=dev), randn(T, D)
    grad = torch.empty(V, D, device=dev)
    wse = ops.embed_workspace(T, V, D, dev)
    if ref is not None:
        emb_r, out_r, dpe_r, grad_r = torch.empty_like(outb), torch.empty_like(outb), torch.empty_like(outb), torch.empty_like(grad)
    ms = time_op(lambda: ops.embed_gather_fwd(table, ids, pe, S, out=outb))
    add("embed_gather_pe_fwd", f"V32000 D4096 T32768 zipf1.1 ({U} distinct)", (U + T) * D * 4 + S * D * 4 + T * 4, ms,
        lambda: ref.pe_add(ref.embed_fwd(table, ids, out=emb_r).view(B, S, D), pe, out=out_r.view(B, S, D)),
        lambda: {"out": bits(outb, out_r)})
    ms = time_op(lambda: ops.embed_sort_tokens(ids, V, D, workspace=wse))
    add("embed_sort_tokens", "T32768", 0, ms)
    ms = time_op(lambda: ops.embed_scatter_bwd(dyb, ids, V, wse, grad=grad))
    add("embed_scatter_bwd", "V32000 D4096 T32768 zipf1.1", T * D * 4 + V * D * 4 + T * 4, ms,
        lambda: ref.embed_bwd(ref.pe_bwd(dyb, dx=dpe_r), ids, V, grad=grad_r),
        # per table row (rel_err_rows_dev): the rms of the whole, mostly empty, table says nothing about a hot row
        lambda: {"grad": rel_err_rows_dev(grad, grad_r)},
        lambda: (lambda e64: ({"grad": rel_err_rows_dev(grad, e64)}, {"grad": rel_err_rows_dev(grad_r, e64)}))(
            torch.zeros(V, D, dtype=torch.float64, device=dev).index_add_(0, ids.long(), dyb.double())))
    del table, outb, dyb, grad
    if ref is not None:
        del emb_r, out_r, dpe_r, grad_r

    # config 4: bias + activation, 32768 x 16384 (2 GiB per buffer)
    R, C = 32768, 16384
    x, dyy = randn(R, C) * 2.0, randn(R, C)
    bias = randn(C) * 0.1
    yb, dxb = torch.empty_like(x), torch.empty_like(x)
    cache = torch.empty(R * C * 4, dtype=torch.uint8, device=dev)
    dbias = torch.empty(C, device=dev)
    wsa = ops.act_bwd_workspace(capi.RELU, R, C, dev)
    n = R * C
    if ref is not None:
        # the reference adds the bias inside its GEMM kernel: its activation kernels start from the biased value
        pre_r = ref.bias_add(x, bias)
        y_r, cache_r, dx_r, dbias_r = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x), torch.empty(C, device=dev)
    cfg4 = "32768x16384 fp32"
    for kind, name in ((capi.RELU, "relu"), (capi.SIGMOID, "sigmoid"), (capi.TANH, "tanh")):
        cache_b = n // 8 if kind == capi.RELU else n * 4
        ms = time_op(lambda: ops.act_fwd(kind, x, bias, y=yb, cache=cache))
        add(f"bias_{name}_fwd", cfg4, n * 8 + cache_b + C * 4, ms,
            lambda: ref.act_fwd(kind, pre_r, y=y_r, cache=cache_r),
            lambda: {"y": bits(yb, y_r)})
        ms = time_op(lambda: ops.act_bwd(kind, dyy, cache, dx=dxb, dbias=dbias, want_dbias=True, workspace=wsa))
        add(f"{name}_bwd_dbias", cfg4, n * 8 + cache_b + C * 4, ms,
            lambda: ref.bias_grad(ref.act_bwd(kind, dyy, cache_r, dx=dx_r), dbias=dbias_r),
            lambda: {"dx": bits(dxb, dx_r), "dbias": rel_err_dev(dbias, dbias_r)},
            lambda: (lambda b64: ({"dbias": rel_err_dev(dbias, b64)}, {"dbias": rel_err_dev(dbias_r, b64)}))(colsum64(dx_r)))
    del x, dyy, yb, dxb, cache
    if ref is not None:
        del pre_r, y_r, cache_r, dx_r

    # beyond the named path (what comes next): GELU epilogue and the optimizer path on the parameters of
    # the chain (embedding table 32000x4096 plus the small groups), one launch for all groups
    R, C = 8192, 16384
    x, dyy, bias = randn(R, C) * 2.0, randn(R, C), randn(C) * 0.1
    yb, dxb, cache = torch.empty_like(x), torch.empty_like(x), torch.empty(R * C * 4, dtype=torch.uint8, device=dev)
    n = R * C
    ms = time_op(lambda: ops.act_fwd(capi.GELU, x, bias, y=yb, cache=cache))
    add("bias_gelu_fwd", "8192x16384 fp32", n * 12 + C * 4, ms)
    ms = time_op(lambda: ops.act_bwd(capi.GELU, dyy, cache, dx=dxb))
    add("gelu_bwd", "8192x16384 fp32", n * 12, ms)
    del x, dyy, yb, dxb, cache
    sizes = [32000 * 4096, 4096, 4096, 4096, 4096, 16384]
    ps, gs = [randn(k) for k in sizes], [randn(k) for k in sizes]
    ms_, vs_ = [torch.zeros(k, device=dev) for k in sizes], [torch.zeros(k, device=dev) for k in sizes]
    total = sum(sizes)
    ms = time_op(lambda: ops.optim_step(capi.OPT_ADAMW, ps, gs, ms_, vs_, lr=1e-3, step=2))
    add("adamw_step_all_groups", "131M params in 6 groups fp32", total * 28, ms)
    res, wsn = torch.empty(3, device=dev), torch.empty(8192, dtype=torch.uint8, device=dev)
    ms = time_op(lambda: ops.grad_norm_clip(gs, 1e9, result=res, workspace=wsn))
    add("grad_norm", "131M gradients in 6 groups fp32", total * 4, ms)
    return out


def reference_kernel_sweep():
    """The reference's own kernels, op by op, on the large fp32 configurations (the launch geometry and
    cache copies of the reference's layer classes); nothing of this library runs here."""
    from oracle import ref
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    randn = lambda *s: torch.randn(*s, generator=g, device=dev)
    out = []

    def add(name, cfg, fn):
        out.append({"kernel": name, "config": cfg, "ms": round(time_op(fn, warmup=1, iters=3), 4)})

    R, D = 65536, 1024
    a, b, dy = randn(R, D), randn(R, D), randn(R, D)
    gamma, beta = torch.rand(D, generator=g, device=dev) + 0.5, randn(D) * 0.1
    s_r, y, xhat, inv = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a), torch.empty(R, device=dev)
    dx, dg, db = torch.empty_like(a), torch.empty(D, device=dev), torch.empty(D, device=dev)
    cfg = "65536x1024 fp32"
    add("ln_residual_fwd", cfg, lambda: ref.ln_fwd(ref.residual_add(a, b, out=s_r), gamma, beta, 1e-5, y=y, xhat=xhat, inv_std=inv))
    add("ln_bwd", cfg, lambda: ref.ln_bwd(dy, xhat, inv, gamma, dx=dx, dgamma=dg, dbeta=db))
    add("ln_bwd_two_grads", cfg, lambda: ref.ln_bwd(ref.residual_add(dy, b, out=s_r), xhat, inv, gamma, dx=dx, dgamma=dg, dbeta=db))
    del a, b, dy, s_r, y, xhat, dx

    V, D, B, S = 32000, 4096, 16, 2048
    T = B * S
    table = randn(V, D) * 0.02
    ids = torch.from_numpy(zipf_ids(np.random.Generator(np.random.Philox(key=1236)), T, V)).to(dev)
    pe = ref.pe_table(S, D).to(dev)
    emb, outb, dpe, dyb = (torch.empty(T, D, device=dev) for _ in range(4))
    dyb.normal_(generator=g)
    grad = torch.empty(V, D, device=dev)
    cfg = "V32000 D4096 T32768 zipf1.1"
    add("embed_gather_pe_fwd", cfg, lambda: ref.pe_add(ref.embed_fwd(table, ids, out=emb).view(B, S, D), pe, out=outb.view(B, S, D)))
    add("embed_scatter_bwd", cfg, lambda: ref.embed_bwd(ref.pe_bwd(dyb, dx=dpe), ids, V, grad=grad))
    del table, emb, outb, dpe, dyb, grad

    R, C = 32768, 16384
    pre, dyy = randn(R, C) * 2.0, randn(R, C)
    y, cache, dx, dbias = torch.empty_like(pre), torch.empty_like(pre), torch.empty_like(pre), torch.empty(C, device=dev)
    cfg = "32768x16384 fp32"
    for kind, name in ((0, "relu"), (1, "sigmoid"), (2, "tanh")):
        add(f"bias_{name}_fwd", cfg, lambda: ref.act_fwd(kind, pre, y=y, cache=cache))
        add(f"{name}_bwd_dbias", cfg, lambda: ref.bias_grad(ref.act_bwd(kind, dyy, cache, dx=dx), dbias=dbias))
    return out


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch, read at run time from the ncu
# summaries under profiles/ (captures of a quarter-size case, or of the full embedding case) and scaled
# by token rows: the traffic of these streaming kernels grows in proportion to the rows.
# (chain op, storage) -> (summary file, kernel-name fragments whose traffic adds up, rows of the captured case)
PROFILE_TRAFFIC = {
    ("embed_gather_pe", "bf16"): ("embedding_kernels_bf16_V32000_D4096_T32768.txt", ["embed_gather_bulk_kernel"], 32768),
    ("ln1_fwd", "bf16"): ("ln_fwd_kernel_bf16_16384x4096.txt", ["ln_fwd_kernel"], 16384),
    ("ln2_fwd", "bf16"): ("ln_fwd_kernel_bf16_16384x4096.txt", ["ln_fwd_kernel"], 16384),
    ("relu_fwd", "bf16"): ("act_relu_kernels_bf16_8192x16384.txt", ["act_fwd_kernel"], 8192),
    ("relu_bwd", "bf16"): ("act_relu_kernels_bf16_8192x16384.txt", ["act_bwd_kernel"], 8192),
    ("ln2_bwd", "bf16"): ("ln_bwd_pipe_kernel_bf16_16384x4096.txt", ["ln_bwd_pipe_kernel"], 16384),
    ("ln1_bwd", "bf16"): ("ln_bwd_pipe_kernel_two_grads_bf16_16384x4096.txt", ["ln_bwd_pipe_kernel"], 16384),
    ("embed_scatter", "bf16"): ("embedding_kernels_bf16_V32000_D4096_T32768.txt",
                                ["scatter_rows_bulk_kernel", "combine_long_kernel"], 32768),
    ("embed_gather_pe", "fp32"): ("embedding_kernels_fp32_V32000_D4096_T32768.txt", ["embed_gather_kernel"], 32768),
    ("embed_scatter", "fp32"): ("embedding_kernels_fp32_V32000_D4096_T32768.txt",
                                ["scatter_rows_bulk_kernel", "combine_long_kernel"], 32768),
}
NCU_TRAFFIC_NOTE = ("ncu dram__bytes_read+write per launch, parsed from profiles/*.txt (a quarter-size or full-size "
                    "capture) and scaled by rows; writes still in L2 when the kernel ends are not counted by ncu, "
                    "so it can read below the algorithmic bytes")
_UNIT_BYTES = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}


def parse_profile(path):
    """[(kernel name, {"dram read": bytes, "dram write": bytes, "duration": us})] of one summary file."""
    kernels = []
    for line in Path(path).read_text().splitlines():
        if line.startswith("kernel:"):
            kernels.append((line.split(":", 1)[1].strip(), {}))
            continue
        if not kernels or not line.startswith("  "):
            continue
        parts = line.split()
        for key in ("dram read", "dram write", "duration"):
            words = key.split()
            if parts[:len(words)] == words and len(parts) == len(words) + 2:
                value, unit = float(parts[-2]), parts[-1]
                if key == "duration":
                    kernels[-1][1][key] = value * {"ns": 1e-3, "us": 1.0, "ms": 1e3}.get(unit, 1.0)
                elif unit in _UNIT_BYTES:
                    kernels[-1][1][key] = value * _UNIT_BYTES[unit]
    return kernels


def ncu_traffic(op, storage, rows):
    """DRAM bytes per launch of a chain op on `rows` token rows, or None where no capture covers it."""
    entry = PROFILE_TRAFFIC.get((op, storage))
    if entry is None:
        return None
    file, fragments, captured_rows = entry
    path = ROOT / "profiles" / file
    if not path.exists():
        return None
    total = 0.0
    for fragment in fragments:
        hits = [m for name, m in parse_profile(path) if fragment in name and "dram read" in m and "dram write" in m]
        if not hits:
            return None
        total += hits[0]["dram read"] + hits[0]["dram write"]
    return int(total / captured_rows * rows)


# --------------------------------------------------------------------------- small cases for ncu
def profile_case(name):
    """One kernel on a case sized for an ncu capture (inputs above L2, well under 2 GB held),
    three calls.  `python bench.py --case NAME`; NAME is one of PROFILE_CASES."""
    from dl_cuda_b200 import capi, ops
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    randn = lambda *s: torch.randn(*s, generator=g, device=dev)
    kind, storage = name.rsplit("_", 1)
    dt = torch.bfloat16 if storage == "bf16" else torch.float32
    if kind in ("ln_fwd", "ln_bwd", "ln_bwd2"):
        R, D = (16384, 4096) if storage == "bf16" else (32768, 1024)
        a, b, dy = randn(R, D).to(dt), randn(R, D).to(dt), randn(R, D).to(dt)
        gamma, beta = torch.rand(D, generator=g, device=dev) + 0.5, randn(D) * 0.1
        y, xhat, inv = torch.empty_like(a), torch.empty_like(a), torch.empty(R, device=dev)
        dx, dg, db = torch.empty_like(a), torch.empty(D, device=dev), torch.empty(D, device=dev)
        ws = ops.ln_bwd_workspace(R, D, dev)
        ops.ln_residual_fwd(a, b, gamma, beta, 1e-5, y=y, xhat=xhat, inv_std=inv)
        for _ in range(3):
            if kind == "ln_fwd":
                ops.ln_residual_fwd(a, b, gamma, beta, 1e-5, y=y, xhat=xhat, inv_std=inv)
            else:
                ops.ln_bwd(dy, b if kind == "ln_bwd2" else None, xhat, inv, gamma, dx=dx, dgamma=dg, dbeta=db,
                           workspace=ws)
    elif kind in ("relu", "tanh"):
        R, C = 8192, 16384
        k = capi.RELU if kind == "relu" else capi.TANH
        x, dy, bias = (randn(R, C) * 2).to(dt), randn(R, C).to(dt), randn(C) * 0.1
        y, dx = torch.empty_like(x), torch.empty_like(x)
        cache, dbias = ops.act_cache(k, x), torch.empty(C, device=dev)
        ws = ops.act_bwd_workspace(k, R, C, dev)
        for _ in range(3):
            ops.act_fwd(k, x, bias, y=y, cache=cache)
            ops.act_bwd(k, dy, cache, dx=dx, dbias=dbias, want_dbias=True, workspace=ws)
    elif kind == "embed":
        V, D, T, S = 32000, 4096, 32768, 2048
        table = (randn(V, D) * 0.02).to(dt)
        ids = torch.from_numpy(zipf_ids(np.random.Generator(np.random.Philox(key=5)), T, V)).to(dev)
        pe, out, dy = ops.pe_table(S, D).to(dev), torch.empty(T, D, device=dev, dtype=dt), randn(T, D).to(dt)
        grad, ws = torch.empty(V, D, device=dev), ops.embed_workspace(T, V, D, dev)
        for _ in range(3):
            # both forms of the gather and of the scatter-add, on the same buffers: seven launches per round
            for form in (1, 2):  # rows in registers, bulk-copy pipeline
                capi.set_option("gather_variant", form)
                ops.embed_gather_fwd(table, ids, pe, S, out=out)
            capi.set_option("gather_variant", 0)
            ops.embed_sort_tokens(ids, V, D, workspace=ws)
            for form in (1, 2):
                capi.set_option("scatter_variant", form)
                ops.embed_scatter_bwd(dy, ids, V, ws, grad=grad)
            capi.set_option("scatter_variant", 0)
    elif kind == "peer":
        # The kernels of the peer-memory exchange as rank 0 of 8 runs them, with the seven peers' buffers
        # standing in on this one GPU (so the "remote" stores are local: this shows the kernels, not NVLink).
        world, V, D = 8, 32000, 4096
        T = 32768 // world
        Tg = T * world
        ids_all = torch.cat([torch.from_numpy(zipf_ids(np.random.Generator(np.random.Philox(key=1234 + r)), T, V))
                             for r in range(world)]).to(dev)
        dx = randn(T, D).to(dt)
        small = randn(4 * D + 16384)
        ws_global = ops.embed_workspace(Tg, V, D, dev)
        cap = (min(V, Tg) + world - 1) // world
        flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(world)]
        recv = torch.zeros(world * cap * D, device=dev)
        mine, theirs = torch.zeros(V, D, device=dev), torch.zeros(V, D, device=dev)
        small_recv = torch.zeros(world * small.numel(), device=dev)
        stage = torch.zeros(world * cap * D, dtype=torch.bfloat16, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        group = ops.peer_group(world, 0, cap, [f.data_ptr() for f in flags], [recv.data_ptr()] * world,
                               [mine.data_ptr()] + [theirs.data_ptr()] * (world - 1), status,
                               [small_recv.data_ptr()] * world, small.numel(), 1000, stage=[stage.data_ptr()] * world)
        rank_plan = ops.embed_rank_plan_workspace(V, T, D, dev)
        small_out = torch.empty_like(small)
        for step in range(1, 4):
            ops.embed_sort_tokens(ids_all, V, D, workspace=ws_global)
            ops.embed_rank_plan(ws_global, Tg, T, world, 0, V, D, rank_plan=rank_plan)
            ops.embed_scatter_bwd_peer(dx, ws_global, Tg, rank_plan, T, group, small, min(V, Tg), V, 0, step, clear_unused=1)
            ops.embed_reduce_broadcast_peer(rank_plan, T, group, small_out, V, D, capi.dtype_of(dx), 3, 0, 1, step)
    elif kind == "optim":
        # AdamW over six groups of 8 Mi parameters, then the gradient norm + clip (fp32 only)
        sizes = [8 << 20] * 6
        params = [randn(n) for n in sizes]
        grads = [randn(n) for n in sizes]
        m = [torch.zeros(n, device=dev) for n in sizes]
        v = [torch.zeros(n, device=dev) for n in sizes]
        result = torch.empty(3, device=dev)
        for step in range(1, 4):
            ops.grad_norm_clip(grads, 1.0, result=result)
            ops.optim_step(capi.OPT_ADAMW, params, grads, m, v, lr=1e-3, step=step)
    else:
        raise SystemExit(f"unknown case {name}; choose from {PROFILE_CASES}")
    torch.cuda.synchronize()
    print(json.dumps({"case": name, "launches": int(capi.lib().dlb_launch_count()),
                      "pipeline_timeouts": capi.pipeline_timeouts()}))


PROFILE_CASES = [f"{k}_{s}" for k in ("ln_fwd", "ln_bwd", "ln_bwd2", "relu", "tanh", "embed") for s in ("fp32", "bf16")]
PROFILE_CASES += ["optim_fp32", "peer_bf16"]


# --------------------------------------------------------------------------- main
def run_timed(step, dist: Dist, steps, warmup, drain=None):
    for _ in range(warmup):
        step()
    dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    if drain is not None:
        drain()  # work the steps left on other streams belongs to the timed region
    stop.record()
    dist.barrier()
    return dist.max_float(start.elapsed_time(stop))


REPEATS = 7  # timed regions of K steps each; the median is reported


def run_repeats(step, dist: Dist, steps, repeats=REPEATS, drain=None):
    """`repeats` back-to-back timed regions of `steps` steps (each: barrier + synchronize on both sides,
    CUDA events, max over ranks).  Returns the per-step times in ms, sorted."""
    return sorted(run_timed(step, dist, steps, 0, drain) / steps for _ in range(repeats))


def capi_timeouts() -> int:
    from dl_cuda_b200 import capi
    return capi.pipeline_timeouts()


def median(values):
    return float(np.median(values))


def print_table(path):
    """Markdown tables of a recorded bench line (`python bench.py --table FILE`): the chain's ops and the
    per-kernel sweep with the reference columns.  The tables in the design notes are this output."""
    line = [json.loads(l) for l in Path(path).read_text().splitlines() if l.startswith("{")][-1]
    peak = line["roofline"]["peak"]
    print(f"N={line['n_gpus']} {line['dtype']}: {line['ms_per_step']:.4f} ms/step = {line['value'] / 1e6:.2f} M tokens/s "
          f"(min {line['value_min'] / 1e6:.2f}, max {line['value_max'] / 1e6:.2f}); e2e {line['e2e']['ms_per_step']:.4f} ms = "
          f"{line['e2e']['value'] / 1e6:.2f} M tokens/s; chain {line['chain_gbs']:.0f} GB/s = "
          f"{line['chain_gbs'] / peak:.3f} of {peak:.1f}; clocks {line['clocks']}")
    if "chain_fp32" in line:
        c = line["chain_fp32"]
        print(f"fp32 chain: {c['ms_per_step']:.4f} ms/step = {c['value'] / 1e6:.2f} M tokens/s, {c['chain_gbs']:.0f} GB/s")
    print("\n| chain op | ms | algorithmic GB/s | of measured peak | ncu DRAM bytes / algorithmic |")
    print("|---|---|---|---|---|")
    for op in line["chain_ops"]:
        if op["gbs"] is None:
            print(f"| {op['op']} | {op['ms']:.4f} | — | — | — |")
        else:
            ratio = f"{op['ncu_traffic'] / op['bytes']:.2f}" if op.get("ncu_traffic") else "—"
            print(f"| {op['op']} | {op['ms']:.4f} | {op['gbs']:.0f} | {op['frac']:.3f} | {ratio} |")
    if "kernels_fp32" in line:
        print("\n| kernel | config | ms | GB/s | of measured peak | reference ms | speed-up | max rel. error vs reference | "
              "vs fp64: ours / reference |")
        print("|---|---|---|---|---|---|---|---|---|")
        for k in line["kernels_fp32"]:
            ref = (f"{k['ref_ms']:.4f} | {k['speedup_vs_ref']:.2f}x | "
                   f"{'bit-exact' if k.get('bit_exact_vs_ref') else format(k.get('max_rel_err_vs_ref', float('nan')), '.2g')}"
                   if "ref_ms" in k else "— | — | —")
            if "err_vs_fp64" in k:
                ref += f" | {max(k['err_vs_fp64'].values()):.2g} / {max(k['ref_err_vs_fp64'].values()):.2g}"
            else:
                ref += " | —"
            gbs = f"{k['gbs']:.0f} | {k['frac_measured']:.3f}" if k.get("gbs") else "— | —"
            print(f"| {k['kernel']} | {k['config']} | {k['ms']:.4f} | {gbs} | {ref} |")


def main():
    if len(sys.argv) == 3 and sys.argv[1] == "--table":
        print_table(sys.argv[2])
        return
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    ap.add_argument("--tokens", type=int, default=BATCH * SEQ, help="global token rows (default: batch 8 x seq 4096)")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="N > 1: how the embedding-table gradient is exchanged (default: the library's peer-memory kernels)")
    ap.add_argument("--clear", choices=["incremental", "fused", "early"], default="incremental",
                    help="N > 1, peer exchange: the table rows no rank uses are cleared inside the push kernel, only "
                         "those the previous step wrote (incremental) or all of them (fused), or all of them early on "
                         "the second stream beside the compute kernels")
    ap.add_argument("--no-split-push", action="store_true",
                    help="N > 1, peer exchange: sums and pushes in stream order instead of overlapped on two streams")
    ap.add_argument("--plan-beside-gather", action="store_true",
                    help="N = 1: start the sorted-segment plan on the second stream at the start of the step (beside the "
                         "gather) instead of after the gather")
    ap.add_argument("--shard", choices=["positions", "sequences"], default="positions",
                    help="N > 1: a rank takes a slice of the positions of every sequence (default) or whole sequences")
    ap.add_argument("--plan-on-main", action="store_true",
                    help="build the sorted-segment plan on the main stream (no second stream in the headline pass)")
    ap.add_argument("--skip-kernels", action="store_true", help="skip the per-kernel fp32 sweep")
    ap.add_argument("--skip-cpu", action="store_true",
                    help="skip the baseline legs (the single-threaded host loops and the reference-kernel columns)")
    ap.add_argument("--skip-fp32-chain", action="store_true", help="N=1: skip the fp32-storage run of the chain")
    ap.add_argument("--skip-overlapped", action="store_true",
                    help="N > 1: skip the extra figure with the exchange of a step beside the next step's forward pass")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="kernel-variant override for A/B measurements (dlb_set_option), may be repeated")
    ap.add_argument("--case", default=None, help="run one small kernel case (for ncu) and exit: " + ", ".join(PROFILE_CASES))
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.option and args.impl == "native":
        from dl_cuda_b200 import capi
        for item in args.option:
            name, value = item.split("=", 1)
            capi.set_option(name, int(value))
    if args.case:
        return profile_case(args.case)

    dist = Dist()
    if dist.world != args.gpus and dist.world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {dist.world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")

    if args.impl == "reference":
        return main_reference(args, dist)

    dist.init()
    peak, peak_kind = measured_peak()
    n = dist.world
    from dl_cuda_b200.sharding import shard_rows
    # Which token rows a rank takes: the same slice of positions of every sequence (a rank then reads 1/N of the
    # positional-encoding table, each row shared by all sequences), or whole sequences.
    by_position = (n > 1 and args.shard == "positions" and args.tokens % SEQ == 0 and SEQ % n == 0)
    if by_position:
        from dl_cuda_b200.sharding import shard_positions
        first_position, seq_local, tokens_local = shard_positions(args.tokens // SEQ, SEQ, n, dist.rank)
    else:
        _, tokens_local = shard_rows(args.tokens, n, dist.rank, SEQ if args.tokens % (SEQ * n) == 0 else 1)
        first_position, seq_local = 0, SEQ
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    chain = Chain(tokens_local, seq_local, D_MODEL, D_FF, VOCAB, dtype, seed=1234 + dist.rank, dist=dist,
                  exchange=args.exchange, clear=args.clear, split_push=not args.no_split_push,
                  plan_after_gather=not args.plan_beside_gather, first_position=first_position, seq_total=SEQ)
    lib = chain.lib
    chain.plan_on_main = args.plan_on_main

    parity = None
    if dist.active:
        # Untimed: one step checked against the single-rank gradient of all tokens, on every rank.
        parity = chain.verify()
        ok = (parity["max_rel_err_table_grad"] <= parity["tolerance"] and parity["max_rel_err_small_grads"] <= parity["tolerance"]
              and parity["ranks_bit_identical"] and parity["status_bits"] == 0)
        if not ok:
            if dist.rank == 0:
                print(json.dumps({"impl": "native", "n_gpus": n, "parity_check": parity, "error": "parity check failed"}))
            dist.finish()
            raise SystemExit(3)

    # device-resident run: the headline `value` (no events between the kernels)
    for _ in range(args.warmup):
        chain.step()
    dist.barrier()
    launches0 = lib.dlb_launch_count()
    sampler = ClockSampler(torch.cuda.current_device())
    with sampler:
        step_ms = run_repeats(chain.step, dist, args.steps)
    launches = (lib.dlb_launch_count() - launches0) // REPEATS
    ms_per_step = median(step_ms)
    tokens_per_s = args.tokens / (ms_per_step / 1e3)

    # the same K steps once more with an event after every op: per-op device time
    marks_all = []

    def step_marked():
        marks = []
        chain.step(marks=marks)
        marks_all.append(marks)

    marked_ms = run_timed(step_marked, dist, args.steps, 1) / args.steps
    marks_all = marks_all[-args.steps:]

    # per-op device time from the events recorded inside the timed region
    op_ms = {name: 0.0 for name in Chain.OPS}
    for marks in marks_all:
        for i, name in enumerate(Chain.OPS):
            op_ms[name] += marks[i].elapsed_time(marks[i + 1])
    op_ms = {k: v / len(marks_all) for k, v in op_ms.items()}
    op_bytes = chain.bytes_per_op()
    ops_report = []
    for name in Chain.OPS:
        gbs = op_bytes[name] / op_ms[name] / 1e6 if op_ms[name] > 0 and op_bytes[name] else None
        ops_report.append({"op": name, "ms": round(op_ms[name], 4), "bytes": int(op_bytes[name]),
                           "gbs": None if gbs is None else round(gbs, 1),
                           "frac": None if gbs is None else round(gbs / peak, 4),
                           "ncu_traffic": ncu_traffic(name, args.dtype, tokens_local) if n == 1 or "embed" not in name
                           else None})
    dominant = max((o for o in ops_report if o["gbs"]), key=lambda o: o["ms"])

    # end to end: ids from pinned host memory in, parameter gradients out, every step
    e2e_step = lambda: chain.step(copy_inputs=True, lagged=True)
    run_timed(e2e_step, dist, args.warmup, 0, chain.readback.drain)
    e2e_all = run_repeats(e2e_step, dist, args.steps, drain=chain.readback.drain)
    e2e_ms = median(e2e_all)
    # the same with the host waiting for every step's result before it queues the next step
    run_timed(lambda: chain.step(copy_inputs=True), dist, 2, 0)
    strict_ms = median(run_repeats(lambda: chain.step(copy_inputs=True), dist, args.steps, repeats=3))
    e2e = {"value": args.tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "value_min": args.tokens / (e2e_all[-1] / 1e3), "value_max": args.tokens / (e2e_all[0] / 1e3),
           "h2d_bytes_per_step": int(chain.h_ids.numel() * 4 * n),
           "d2h_bytes_per_step": int(chain.h_result.numel() * 4 * n),
           "host_waits_every_step": {"value": args.tokens / (strict_ms / 1e3), "ms_per_step": round(strict_ms, 4)},
           "what": "per step: token ids copied from pinned host memory, the chain through the C ABI, "
                   "gamma/beta/bias gradients copied back to pinned host memory and read there. The host reads the "
                   "result of step i after it has queued step i+1 (one step of lag, as a training loop that logs "
                   "its loss does); each region ends when its last result has been read. host_waits_every_step: "
                   "the same with a host synchronisation after every step"}

    result = {
        "metric": "tokens/s", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "impl": "native",
        "value_min": args.tokens / (step_ms[-1] / 1e3), "value_max": args.tokens / (step_ms[0] / 1e3),
        "repeats": REPEATS, "ms_per_step_all": [round(v, 4) for v in step_ms],
        "timing": f"median of {REPEATS} timed regions of {args.steps} steps each (gpu_launches: per region)",
        "options": args.option,
        "config": {"workload": "transformer-block non-GEMM chain fwd+bwd (embed+PE, LN+residual x2, bias+ReLU, "
                               "scatter-add), token-sharded",
                   "batch": BATCH, "seq_len": SEQ, "d_model": D_MODEL, "d_ff": D_FF, "vocab": VOCAB,
                   "global_tokens": args.tokens, "tokens_per_gpu": tokens_local, "ids": "zipf(1.1)",
                   "parallelism": (f"token rows / {n}" + (f": positions {first_position}..{first_position + seq_local - 1} of "
                                                             f"every sequence on rank 0" if by_position else
                                                             ": whole sequences per rank" if n > 1 else "")), "l2": "inputs larger than L2 (about 10 GB touched per step)"},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": sampler.summary(),
        "roofline": {"bound": "hbm", "kernel": dominant["op"], "achieved": dominant["gbs"], "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": dominant["frac"],
                     "frac_of_nominal_8000": round(dominant["gbs"] / NOMINAL_HBM_GBS, 4),
                     "algorithmic_bytes": dominant["bytes"],
                     "traffic": ncu_traffic(dominant["op"], args.dtype, tokens_local),
                     "traffic_source": NCU_TRAFFIC_NOTE},
        "chain_ops": ops_report, "chain_ops_ms_per_step": round(marked_ms, 4),
        "chain_ops_note": "per-op times come from a second pass of the same K steps with a CUDA event after "
                          "every op (ops serialised on one stream); the headline pass has no events and "
                          "builds the token plan on a side stream",
        "chain_bytes_per_step": int(sum(op_bytes.values()) * n),
        "chain_gbs": round(sum(op_bytes.values()) * n / ms_per_step / 1e6, 1),
    }
    if capi_timeouts():
        raise SystemExit("a pipeline wait gave up during the run: the measurement is void")
    if dist.active:
        result["config"]["table_grad_exchange"] = chain.exchange_note
        result["parity_check"] = parity
        if chain.peer is not None:
            gave_up = chain.peer.timed_out()
            if gave_up:
                raise SystemExit(f"peer exchange status {gave_up:#x} (a wait gave up or the receive area was too small): "
                                 "the measurement is void")
        # The second figure: the exchange of step i beside the forward pass of step i+1 (every exchange buffer
        # twice).  Not the headline: a training step's optimizer would have to wait for the exchange.
        try:
            overlapped = chain.peer is not None and not args.skip_overlapped and chain.enable_overlap()
        except Exception as exc:  # the second set of symmetric buffers could not be set up
            overlapped = False
            result["value_overlapped"] = {"error": f"{type(exc).__name__}: {exc}"}
        if overlapped:
            check = chain.verify_overlapped()
            good = (check["max_rel_err_table_grad"] <= check["tolerance"] and check["status_bits_clear"]
                    and check["max_rel_err_small_grads"] <= check["tolerance"])
            if good:
                run_timed(chain.step_overlapped, dist, args.warmup, 0, chain.drain_overlapped)
                ov_ms = run_repeats(chain.step_overlapped, dist, args.steps, drain=chain.drain_overlapped)
                ms_ov = median(ov_ms)
                status = 0
                for cur in chain.sets:
                    status |= cur["peer"].timed_out()
                good = status == 0 and capi_timeouts() == 0
            if good:
                result["value_overlapped"] = {
                    "value": args.tokens / (ms_ov / 1e3), "unit": "tokens/s", "ms_per_step": round(ms_ov, 4),
                    "value_min": args.tokens / (ov_ms[-1] / 1e3), "value_max": args.tokens / (ov_ms[0] / 1e3),
                    "parity_check": check,
                    "what": "not the critical-path figure: the table-gradient exchange of step i runs on a stream of its "
                            "own beside the forward pass of step i+1 (every exchange buffer and the dense table twice); "
                            "each timed region ends when its last exchange has ended"}
            else:
                result["value_overlapped"] = {"error": "the overlapped steps failed their check", "parity_check": check}
    del chain
    torch.cuda.empty_cache()
    if n == 1 and args.dtype == "bf16" and not args.skip_fp32_chain:
        # The like-for-like figure against the reference arm (which is fp32: the reference has no bf16):
        # the same chain with fp32 storage, same steps and warm-up.
        chain32 = Chain(tokens_local, SEQ, D_MODEL, D_FF, VOCAB, torch.float32, seed=1234, dist=dist)
        run_timed(chain32.step, dist, args.warmup, 0)
        ms32_all = run_repeats(chain32.step, dist, args.steps)
        ms32 = median(ms32_all)
        bytes32 = sum(chain32.bytes_per_op().values())
        e2e32_step = lambda: chain32.step(copy_inputs=True, lagged=True)
        run_timed(e2e32_step, dist, args.warmup, 0, chain32.readback.drain)
        e2e32 = median(run_repeats(e2e32_step, dist, args.steps, drain=chain32.readback.drain))
        result["chain_fp32"] = {"ms_per_step": round(ms32, 4), "value": args.tokens / (ms32 / 1e3), "unit": "tokens/s",
                                "value_min": args.tokens / (ms32_all[-1] / 1e3),
                                "value_max": args.tokens / (ms32_all[0] / 1e3),
                                "e2e_value": args.tokens / (e2e32 / 1e3),
                                "chain_bytes_per_step": int(bytes32), "chain_gbs": round(bytes32 / ms32 / 1e6, 1),
                                "what": "the same chain with fp32 storage: the figure to hold against the reference "
                                        "arm, whose kernels are fp32"}
        if lib.dlb_launch_count() and capi_timeouts():
            raise SystemExit("a pipeline wait gave up during the fp32 chain: the measurement is void")
        del chain32
        torch.cuda.empty_cache()
    if dist.rank == 0 and n == 1:
        if not args.skip_kernels:
            # with the baseline legs on, the reference's own kernels are timed beside each large-config kernel
            result["kernels_fp32"] = kernel_sweep(peak, with_reference=not args.skip_cpu)
        if not args.skip_cpu:
            result["cpu_baseline"] = cpu_baseline()
    dist.barrier()
    if dist.rank == 0:
        print(json.dumps(result))
    dist.finish()


def main_reference(args, dist: Dist):
    """Reference arm: the reference's unmodified CUDA kernels (it has no CPU implementation and
    no bf16 or multi-GPU path) on the fp32 version of the same chain, one GPU, rank 0 only."""
    if dist.rank != 0:
        return
    from oracle import ref
    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libref_shim.so was not built "
                          "(the reference checkout was absent at build time)"}))
        return
    torch.cuda.set_device(dist.local_rank)
    one = Dist()
    one.active = False
    chain = ReferenceChain(args.tokens, SEQ, D_MODEL, D_FF, VOCAB, seed=1234)
    sampler = ClockSampler(torch.cuda.current_device())
    for _ in range(args.warmup):
        chain.step()
    torch.cuda.synchronize()
    with sampler:
        total_ms = run_timed(chain.step, one, args.steps, 0)
    ms = total_ms / args.steps
    # end to end, the way the native arm measures it: the host reads a step's result one step late
    drain = lambda: chain.readback.drain() if hasattr(chain, "readback") else None
    e2e_ms = run_timed(lambda: chain.step(copy_inputs=True, lagged=True), one, args.steps, 1, drain) / args.steps
    value = args.tokens / (ms / 1e3)
    h2d, d2h = int(chain.h_ids.numel() * 4), int(chain.h_result.numel() * 4)
    del chain
    torch.cuda.empty_cache()
    sweep = None if args.skip_kernels else reference_kernel_sweep()
    print(json.dumps({
        "impl": "reference", "metric": "tokens/s", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": "transformer-block non-GEMM chain fwd+bwd through the reference's own CUDA kernels "
                               "(fp32: the reference has no bf16; single GPU: it has no multi-GPU path)",
                   "batch": BATCH, "seq_len": SEQ, "d_model": D_MODEL, "d_ff": D_FF, "vocab": VOCAB,
                   "global_tokens": args.tokens, "ids": "zipf(1.1)",
                   "l2": "inputs larger than L2"},
        "e2e": {"value": args.tokens / (e2e_ms / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": 0, "kind": "reference",
                         "sample": "the reference's CUDA kernels built for sm_100 on the same B200 "
                                   "(the reference has no CPU implementation of this path)"},
        "clocks": sampler.summary(),
        "kernels_fp32_reference": sweep,
        "kernels_note": "per-op times of the reference's kernels on the large fp32 configurations; the bias add is "
                        "inside the reference's GEMM kernel and is not timed",
    }))


if __name__ == "__main__":
    main()
