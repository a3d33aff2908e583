"""Headline benchmark: Gemma-3 4B pre-training step throughput (tokens/s over the whole job).

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Config: Gemma-3 4B, 34 layers, d_model 2560, 8 q / 4 kv heads, head_dim 256, GeGLU
10240, vocab 262208 tied, 5:1 local:global attention with window 1024, seq 8192, micro-batch 2 per
GPU, bf16 compute with fp32 master weights / reduction, selective activation recomputation, AdamW
without decay on embeddings and norms, sharded data parallel over N GPUs (weak scaling).  Data:
uniform-random tokens packed into geometric(mean 1500) documents with a same-document mask; weights
are randomly initialised.

Timing: W untimed steps, then K steps between two CUDA events bracketed by barrier + synchronize;
the reported time is the maximum over ranks.  The device-timed loop reads batches that already sit
on the GPU; the end-to-end loop goes through ``Trainer.train_step`` with pinned host batches (H2D
every step) and reads the loss back to the host every step.  A step touches tens of GB, far more
than the 126 MB L2, so no explicit flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL, FLAVOR, SEQ, MICRO_BATCH = "gemma3", "4B", 8192, 2
ADAMW_GROUPS = [
    {"opt_class": "torch.optim.AdamW",
     "opt_cfg": {"lr": 3e-4, "betas": (0.9, 0.95), "weight_decay": 0.1, "eps": 1e-8, "fused": True},
     "min_dim": 2, "exclude_names": ["tok_embeddings"]},
    {"opt_class": "torch.optim.AdamW",
     "opt_cfg": {"lr": 3e-4, "betas": (0.9, 0.95), "weight_decay": 0.0, "eps": 1e-8, "fused": True},
     "min_dim": 0},
]


# --------------------------------------------------------------------------- helpers
class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi during a region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.path = gpu_index, None, f"/tmp/clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "reasons": sorted(reasons)}


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1 or n_gpus > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return world, int(os.environ.get("RANK", "0")), local_rank


def timed_region(fn, steps: int, world: int) -> float:
    """Milliseconds for ``steps`` calls of ``fn`` on this rank's stream, max over ranks."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def host_batches(n: int, rank: int, vocab: int, pin: bool = True):
    from maester_b200.datasets.synthetic import SyntheticLoader
    # packed documents with per-document positions: both arms get document_ids AND position_ids, as the reference's
    # trainer passes both to the model when the batch has them (train.py:324-362 of the reference)
    loader = SyntheticLoader(MICRO_BATCH, SEQ, vocab, "geometric:1500", seed=0, rank=rank, pin=pin,
                             with_position_ids=True)
    return [next(loader) for _ in range(n)]


def emit(args, world, value, ms_per_step, e2e, clocks, launches, impl, extra=None):
    global_batch = MICRO_BATCH * world
    line = {
        "metric": "tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": impl,
        "config": {"model": "gemma3-4B", "global_batch": global_batch, "seq_len": SEQ,
                   "parallelism": f"dp{world}" if world > 1 else "single",
                   "micro_batch_per_gpu": MICRO_BATCH,
                   "activation_checkpointing": ("selective(op): the reference's per-op policy under torch.compile"
                                                if impl == "reference" else
                                                "selective(op): q/k normalisation + rotation recomputed in backward"),
                   "optimizer": "AdamW (no decay on embeddings/norms), fp32 master",
                   "l2": "per-step working set >> 126 MB L2, no flush needed"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
    }
    if extra:
        line["config"].update(extra)
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- this framework
def run_ours(args):
    world, rank, local_rank = dist_setup(args.gpus)
    from maester_b200.config import Config
    from maester_b200.log_utils import init_logger
    from maester_b200.ops import cuda as C
    from maester_b200.trainer import Trainer

    init_logger()
    cfg = Config(model_name=MODEL, flavor=args.flavor, seq_len=SEQ, train_batch_size=MICRO_BATCH,
                 data_parallel_shard_degree=world, ac_mode=args.ac, selective_ac_option="op",
                 optimizer_groups=ADAMW_GROUPS, scheduler="linear_warmup_cosine", warmup_steps=100,
                 train_num_steps=10_000, enable_checkpoint=False, synthetic_data=True,
                 fused_collectives=not args.no_fused_collectives)
    trainer = Trainer(cfg)
    vocab = trainer.model_args.vocab_size
    pool = host_batches(4, rank, vocab)
    dev_pool = [trainer.to_device(b) for b in pool]
    torch.cuda.synchronize()

    for i in range(args.warmup):
        trainer.train_step(dev_pool[i % len(dev_pool)])
    C.check_status()

    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = C.launch_count
    ms = timed_region(lambda i: trainer.train_step(dev_pool[i % len(dev_pool)]), args.steps, world)
    launches = C.launch_count - l0
    clocks = sampler.stop()
    C.check_status()

    # end to end: pinned host batch -> device every step, loss read back every step
    losses = []

    def e2e_step(i):
        loss = trainer.train_step(pool[i % len(pool)])
        losses.append(loss.item())

    ms_e2e = timed_region(e2e_step, args.steps, world)
    C.check_status()
    tokens = MICRO_BATCH * SEQ * world * args.steps
    h2d = sum(v.numel() * v.element_size() for v in pool[0].values())
    e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": losses[-1]}
    if rank == 0:
        value = tokens / (ms / 1e3)
        extra_mfu = trainer.mfu(value / world)
        sys.stderr.write(f"[bench] {ms / args.steps:.1f} ms/step, {value:,.0f} tok/s, MFU {extra_mfu:.1f}% "
                         f"(of 2.25 PF), e2e {e2e['value']:,.0f} tok/s, loss {losses[-1]:.3f}\n")
        sh = trainer.sharded
        coll = "none (one GPU)"
        if world > 1:
            coll = "nccl" if not (sh and sh.fused) else ("multimem" if sh.symm_grad.multicast_ptr else "peer")
        free, total = torch.cuda.mem_get_info()
        emit(args, world, value, ms / args.steps, e2e, clocks, launches, "maester_b200",
             {"collectives": coll, "resharding": bool(sh is not None and sh.resharded),
              "device_used_gib": round((total - free) / 2**30, 1)})
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- the reference
def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "maester")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/maester is not installed"}))
        return
    # cut_cross_entropy is imported unconditionally by the reference models but is not installable
    # offline; the stand-in only satisfies the import, the run uses enable_cut_cross_entropy=False
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, ref_dir)
    try:
        world, rank, local_rank = dist_setup(args.gpus)
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29534")
            os.environ.setdefault("RANK", "0")
            os.environ.setdefault("WORLD_SIZE", "1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        import torch.nn.functional as F
        from maester.config import Config as RefConfig
        from maester.lr_scheduling import get_lr_scheduler
        from maester.models import (model_name_to_cls, model_name_to_optimizers_builder,
                                    model_name_to_parallelize, models_config)
        from maester.parallelisms import ParallelDims
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
        return

    cfg = RefConfig(model_name=MODEL, flavor=args.flavor, seq_len=SEQ, train_batch_size=MICRO_BATCH,
                    data_parallel_shard_degree=world, data_parallel_replicate_degree=1, tensor_parallel_degree=1,
                    ac_mode=args.ac, selective_ac_option="op", compile=True, enable_cut_cross_entropy=False,
                    optimizer_groups=ADAMW_GROUPS, scheduler="linear_warmup_cosine", warmup_steps=100,
                    train_num_steps=10_000, enable_checkpoint=False, norm_type="compiled_rmsnorm")
    pd = ParallelDims(dp_shard=world, dp_replicate=1, tp=1, ep=1, world_size=world, enable_loss_parallel=False)
    world_mesh = pd.world_mesh
    model_config = models_config[MODEL][args.flavor]
    model_config.norm_type = cfg.norm_type
    model_config.max_seq_len = SEQ
    with torch.device("meta"):
        model = model_name_to_cls[MODEL].from_model_args(model_config)
    model_name_to_parallelize[MODEL](model, world_mesh, pd, cfg)
    model.to_empty(device="cuda")
    model.init_weights()
    optimizers = model_name_to_optimizers_builder[MODEL](model, cfg, pd)
    scheduler = get_lr_scheduler(optimizers, cfg)
    model.train()

    pool = host_batches(4, rank, model_config.vocab_size)
    dev_pool = [{k: v.cuda(non_blocking=True) for k, v in b.items()} for b in pool]
    counter = [0]

    def step(batch, from_host: bool):
        optimizers.zero_grad(set_to_none=True)
        counter[0] += 1
        torch.manual_seed(counter[0] + rank)
        if from_host:
            batch = {k: v.cuda(non_blocking=True) for k, v in batch.items()}
        pred = model(batch["input_ids"], position_ids=batch.get("position_ids"), document_ids=batch["document_ids"])
        loss = F.cross_entropy(pred.flatten(0, 1).float(), batch["labels"].flatten(0, 1))
        del pred
        loss.backward()
        optimizers.step()
        scheduler.step()
        return loss

    for i in range(args.warmup):
        step(dev_pool[i % len(dev_pool)], False)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_region(lambda i: step(dev_pool[i % len(dev_pool)], False), args.steps, world)
    clocks = sampler.stop()
    losses = []
    ms_e2e = timed_region(lambda i: losses.append(step(pool[i % len(pool)], True).item()), args.steps, world)
    tokens = MICRO_BATCH * SEQ * world * args.steps
    h2d = sum(v.numel() * v.element_size() for v in pool[0].values())
    e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": losses[-1]}
    if rank == 0:
        emit(args, world, tokens / (ms / 1e3), ms / args.steps, e2e, clocks, None, "reference",
             {"collectives": "nccl (FSDP2)" if world > 1 else "none (one GPU)",
              "loss": "full logits + F.cross_entropy (cut_cross_entropy cannot be installed offline)"})
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--flavor", default=FLAVOR)
    ap.add_argument("--ac", default="selective")
    ap.add_argument("--no-fused-collectives", action="store_true",
                    help="use NCCL reduce-scatter/all-gather instead of the fused peer-memory optimizer kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    if args.impl == "reference":
        try:
            run_reference(args)
        except Exception as e:  # noqa: BLE001
            import traceback
            traceback.print_exc()
            print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
