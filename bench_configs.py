"""Throughput of the secondary training configurations (the flagship one is ``bench.py``).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29540 \
        bench_configs.py --preset deepseek-moe-ep8 --gpus 8 [--steps 8 --warmup 3] [--ep-peer] [--no-fused-collectives]

Presets (shapes of the reference's headline configurations; synthetic packed data, random-init weights):

* ``gemma3-4b``         Gemma-3 4B, seq 8192, micro-batch 2 per GPU (the configuration of ``bench.py``)
* ``gemma3-1b``         Gemma-3 1B, seq 8192, micro-batch 4 per GPU, data-parallel sharding over all GPUs
* ``llama3-8b-tp2``     Llama-3 8B, seq 8192, micro-batch 2 per data-parallel rank, TP=2 x FSDP
* ``llama3-8b-cp2``     Llama-3 8B, seq 32768, micro-batch 1, context parallel 2 x FSDP
* ``deepseek-moe-ep8``  16-layer DeepSeek-style MoE (64 routed experts, top-6), seq 4096, micro-batch 4 per GPU,
                        expert parallel over all GPUs x FSDP
* ``deepseek-moe-1gpu`` the same MoE block at 6 layers (fits one GPU without expert parallelism), seq 4096, micro-batch 4

Timing as in ``bench.py``: warm-up, then CUDA events around K steps between barriers, max over ranks,
clocks sampled during the timed region; one JSON line from rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

import bench as B

PRESETS = {
    "gemma3-4b": dict(model_name="gemma3", flavor="4B", seq_len=8192, train_batch_size=2),
    "gemma3-1b": dict(model_name="gemma3", flavor="1B", seq_len=8192, train_batch_size=4),
    "gemma3-4b-tp2": dict(model_name="gemma3", flavor="4B", seq_len=8192, train_batch_size=2, tensor_parallel_degree=2),
    "llama3-8b-tp2": dict(model_name="llama3", flavor="8B", seq_len=8192, train_batch_size=2, tensor_parallel_degree=2),
    "llama3-8b-cp2": dict(model_name="llama3", flavor="8B", seq_len=32768, train_batch_size=1, context_parallel_degree=2),
    "deepseek-moe-ep8": dict(model_name="deepseek", flavor="bench16L", seq_len=4096, train_batch_size=4,
                             expert_parallel="world"),
    # the same model over 4 ranks (16 experts per rank): the A/B against the reference where 8-GPU boxes are scarce
    "deepseek-moe-ep4": dict(model_name="deepseek", flavor="bench16L", seq_len=4096, train_batch_size=4,
                             expert_parallel="world"),
    # fp32 master + Adam state + gradient shard: 16 B/parameter, 108 GB per GPU at 4 GPUs (54 GB at 8); the bf16
    # parameters exist per block only while the block runs (resharding mode of the sharding runtime); run it with
    # --ac full on 4 GPUs (the activations of 62 blocks at 8192 tokens would not fit beside the state otherwise)
    "gemma3-27b": dict(model_name="gemma3", flavor="27B", seq_len=8192, train_batch_size=1),
    "deepseek-moe-1gpu": dict(model_name="deepseek", flavor="bench6L", seq_len=4096, train_batch_size=4),
}
# smallest world size whose GPUs hold the configuration (sharded fp32 state + activations within 180 GB each)
MIN_GPUS = {"gemma3-4b-tp2": 2, "llama3-8b-cp2": 4, "deepseek-moe-ep8": 8, "deepseek-moe-ep4": 4, "gemma3-27b": 4}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", required=True, choices=sorted(PRESETS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ac", default="selective")
    ap.add_argument("--ep-peer", action="store_true", help="expert-parallel exchange by peer-memory kernels")
    ap.add_argument("--no-fused-collectives", action="store_true")
    ap.add_argument("--vocab", type=int, default=0, help="override the vocabulary size (0: the flavor's, or 128256)")
    ap.add_argument("--cp-mode", default="alltoall", choices=["alltoall", "ring"], help="context-parallel attention form")
    ap.add_argument("--docs", default=None, help="document lengths of the synthetic data (default geometric:1500; "
                    "the ring form needs 'full': one document per row)")
    ap.add_argument("--reshard", default="default", choices=["default", "never", "always"],
                    help="fsdp_reshard_after_forward")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="'reference': the unmodified reference from baseline/_ref through its own registries")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    if not torch.cuda.is_available():
        print(json.dumps({"preset": a.preset, "unavailable": "no CUDA device"}))
        return
    need = MIN_GPUS.get(a.preset, 1)
    if int(os.environ.get("WORLD_SIZE", a.gpus)) < need:  # refuse before anything is allocated
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"preset": a.preset, "unavailable": f"needs at least {need} GPUs (the preset's parallel degrees, "
                              "or the fp32 state of the whole model, which does not fit the memory of fewer)"}))
        return
    if a.impl == "reference":
        try:
            run_reference(a)
        except Exception as e:  # noqa: BLE001
            import traceback
            traceback.print_exc()
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "preset": a.preset,
                                  "unavailable": f"{type(e).__name__}: {e}"[:400]}), flush=True)
        return
    world, rank, local_rank = B.dist_setup(a.gpus)
    from maester_b200.config import Config
    from maester_b200.datasets.synthetic import SyntheticLoader
    from maester_b200.log_utils import init_logger
    from maester_b200.ops import cuda as C
    from maester_b200.trainer import Trainer

    init_logger()
    p = dict(PRESETS[a.preset])
    ep = p.pop("expert_parallel", None)
    tp, cp = p.get("tensor_parallel_degree", 1), p.get("context_parallel_degree", 1)
    cfg = Config(**p, data_parallel_shard_degree=world // (tp * cp), expert_parallel_degree=world if ep == "world" else 1,
                 ac_mode=a.ac, selective_ac_option="op", optimizer_groups=B.ADAMW_GROUPS, scheduler="linear_warmup_cosine",
                 warmup_steps=100, train_num_steps=10_000, enable_checkpoint=False, synthetic_data=True,
                 synthetic_vocab_size=a.vocab or 128256, fused_collectives=not a.no_fused_collectives,
                 ep_peer_dispatch=a.ep_peer, context_parallel_mode=a.cp_mode, fsdp_reshard_after_forward=a.reshard)
    trainer = Trainer(cfg)
    vocab = trainer.model_args.vocab_size
    mb, seq = cfg.train_batch_size, cfg.seq_len
    docs = a.docs or ("full" if (cp > 1 and a.cp_mode == "ring") else "geometric:1500")
    loader = SyntheticLoader(mb, seq, vocab, docs, seed=0, rank=trainer.dp_rank, pin=True)
    pool = [next(loader) for _ in range(4)]
    dev_pool = [trainer.to_device(b) for b in pool]
    torch.cuda.synchronize()
    for i in range(a.warmup):
        trainer.train_step(dev_pool[i % 4])
    C.check_status()
    sampler = B.ClockSampler(local_rank)
    sampler.start()
    l0 = C.launch_count
    ms = B.timed_region(lambda i: trainer.train_step(dev_pool[i % 4]), a.steps, world)
    launches = C.launch_count - l0
    clocks = sampler.stop()
    C.check_status()
    losses = []

    def e2e_step(i):
        losses.append(trainer.train_step(pool[i % 4]).item())

    ms_e2e = B.timed_region(e2e_step, a.steps, world)
    dp = world // (tp * cp)
    tokens = mb * seq * dp * a.steps
    if rank == 0:
        value = tokens / (ms / 1e3)
        par = "+".join(s for s in (f"dp{dp}" if dp > 1 else "", f"tp{tp}" if tp > 1 else "", f"cp{cp}" if cp > 1 else "",
                                   f"ep{world}" if ep else "") if s) or "single"
        sys.stderr.write(f"[bench_configs] {a.preset}: {ms / a.steps:.1f} ms/step, {value:,.0f} tok/s, "
                         f"MFU {trainer.mfu(value / world):.1f}% (of 2.25 PF)\n")
        print(json.dumps({
            "metric": "tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"preset": a.preset, "model": f"{cfg.model_name}-{cfg.flavor}", "global_batch": mb * dp, "seq_len": seq,
                       "parallelism": par, "ep_exchange": ("peer-memory kernels" if a.ep_peer else "all_to_all") if ep else None,
                       "fused_collectives": not a.no_fused_collectives, "documents": docs,
                       "context_parallel_mode": a.cp_mode if cp > 1 else None,
                       "resharding": bool(trainer.sharded is not None and trainer.sharded.resharded),
                       "peak_allocated_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2),
                       # device-wide (symmetric buffers are not the caching allocator's): used memory at the end
                       "device_used_gib": round((torch.cuda.mem_get_info()[1] - torch.cuda.mem_get_info()[0]) / 2**30, 2)},
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in pool[0].values()),
                    "d2h_bytes_per_step": 4, "last_loss": losses[-1]},
        }), flush=True)


def run_reference(a) -> None:
    """The same preset through the reference's own code: its Config, ParallelDims, model registries, ``parallelize_*``
    (tensor parallel + sequence parallel + loss parallel for Llama, ``parallelize_llama.py:32-181``; expert parallel +
    FSDP2 for DeepSeek, ``parallelize_deepseek.py:264-481``), optimizer builder and LR scheduler, with the loop of its
    ``train.py:314-390`` (loss-parallel context, plain cross-entropy on logits because ``cut_cross_entropy`` cannot be
    installed offline).  Nothing of this framework is on that path except the synthetic batches."""
    import contextlib
    import copy
    import dataclasses

    import torch.distributed as dist

    ref_dir = os.path.join(B.ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "maester")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/maester is not installed"}))
        return
    sys.path.insert(0, os.path.join(B.ROOT, "baseline", "shims"))
    sys.path.insert(0, ref_dir)
    world, rank, local_rank = B.dist_setup(a.gpus)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29535")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import torch.nn.functional as F
    from maester.config import Config as RefConfig
    from maester.lr_scheduling import get_lr_scheduler
    from maester.models import (model_name_to_cls, model_name_to_optimizers_builder, model_name_to_parallelize,
                                models_config)
    from maester.parallelisms import ParallelDims
    from maester_b200.datasets.synthetic import SyntheticLoader
    from torch.distributed.tensor.parallel import loss_parallel

    p = dict(PRESETS[a.preset])
    ep = p.pop("expert_parallel", None)
    tp, cp = p.get("tensor_parallel_degree", 1), p.pop("context_parallel_degree", 1)
    if cp > 1:
        raise NotImplementedError("the reference has no context parallelism (maester/parallelisms/parallel_dims.py:15)")
    name, flavor = p["model_name"], p["flavor"]
    if flavor in models_config[name]:
        model_config = copy.deepcopy(models_config[name][flavor])
    else:
        # a benchmark flavor of this framework (the MoE presets): the same shape in the reference's own dataclasses
        from maester_b200.models import models_config as ours
        mine = ours[name][flavor]
        ref_cls = type(next(iter(models_config[name].values())))
        fields = {f.name for f in dataclasses.fields(ref_cls)}
        kw = {k: v for k, v in dataclasses.asdict(mine).items() if k in fields and k != "moe_args"}
        if "moe_args" in fields:
            from maester.models.moe import MoEArgs as RefMoE
            mf = {f.name for f in dataclasses.fields(RefMoE)}
            kw["moe_args"] = RefMoE(**{k: v for k, v in dataclasses.asdict(mine.moe_args).items() if k in mf})
        model_config = ref_cls(**kw)
    if getattr(model_config, "vocab_size", 0) <= 0:
        model_config.vocab_size = a.vocab or 128256
    dp = world // tp
    note = {}
    for compile_flag in (True, False):
        try:
            cfg = RefConfig(**p, data_parallel_shard_degree=dp, data_parallel_replicate_degree=1,
                            expert_parallel_degree=world if ep == "world" else 1, ac_mode=a.ac, selective_ac_option="op",
                            compile=compile_flag, enable_cut_cross_entropy=False, enable_loss_parallel=True,
                            optimizer_groups=B.ADAMW_GROUPS, scheduler="linear_warmup_cosine", warmup_steps=100,
                            train_num_steps=10_000, enable_checkpoint=False, norm_type="compiled_rmsnorm" if compile_flag else "rmsnorm")
            pd = ParallelDims(dp_shard=dp, dp_replicate=1, tp=tp, ep=world if ep == "world" else 1, world_size=world,
                              enable_loss_parallel=True)
            world_mesh = pd.world_mesh
            mc = copy.deepcopy(model_config)
            if hasattr(mc, "norm_type"):
                mc.norm_type = cfg.norm_type
            mc.max_seq_len = cfg.seq_len
            with torch.device("meta"):
                model = model_name_to_cls[name].from_model_args(mc)
            model_name_to_parallelize[name](model, world_mesh, pd, cfg)
            model.to_empty(device="cuda")
            model.init_weights()
            optimizers = model_name_to_optimizers_builder[name](model, cfg, pd)
            scheduler = get_lr_scheduler(optimizers, cfg)
            model.train()
            dp_rank = world_mesh["dp"].get_local_rank() if pd.dp_enabled else 0
            mb, seq = cfg.train_batch_size, cfg.seq_len
            loader = SyntheticLoader(mb, seq, mc.vocab_size, a.docs or "geometric:1500", seed=0, rank=dp_rank, pin=True)
            pool = [next(loader) for _ in range(4)]
            dev_pool = [{k: v.cuda(non_blocking=True) for k, v in b.items()} for b in pool]
            lp_ctx = loss_parallel if pd.loss_parallel_enabled else contextlib.nullcontext
            counter = [0]

            def step(batch, from_host: bool):
                optimizers.zero_grad(set_to_none=True)
                counter[0] += 1
                torch.manual_seed(counter[0] + dp_rank)
                if from_host:
                    batch = {k: v.cuda(non_blocking=True) for k, v in batch.items()}
                with lp_ctx():
                    pred = model(batch["input_ids"], position_ids=batch.get("position_ids"),
                                 document_ids=batch.get("document_ids"))
                    loss = F.cross_entropy(pred.flatten(0, 1).float(), batch["labels"].flatten(0, 1))
                    del pred
                    loss.backward()
                optimizers.step()
                scheduler.step()
                return loss

            for i in range(a.warmup):
                step(dev_pool[i % 4], False)
            break
        except Exception as e:  # noqa: BLE001  (e.g. a torch.compile failure: the reference's compile=False path is stock too)
            if not compile_flag:
                raise
            note["compile"] = f"compile=True failed ({type(e).__name__}: {str(e)[:120]}); ran with compile=False"
            for v in ("model", "optimizers", "scheduler"):
                locals().pop(v, None)
            torch.cuda.empty_cache()
    sampler = B.ClockSampler(local_rank)
    sampler.start()
    ms = B.timed_region(lambda i: step(dev_pool[i % 4], False), a.steps, world)
    clocks = sampler.stop()
    losses = []

    def e2e_step(i):
        l = step(pool[i % 4], True).detach()
        l = l.full_tensor() if hasattr(l, "full_tensor") else l
        losses.append(float(l.float().mean().item()))

    ms_e2e = B.timed_region(e2e_step, a.steps, world)
    tokens = mb * seq * dp * a.steps
    if rank == 0:
        par = "+".join(x for x in (f"dp{dp}" if dp > 1 else "", f"tp{tp}" if tp > 1 else "", f"ep{world}" if ep else "") if x) or "single"
        print(json.dumps({
            "metric": "tokens_per_sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "impl": "reference",
            "config": {"preset": a.preset, "model": f"{name}-{flavor}", "global_batch": mb * dp, "seq_len": seq,
                       "parallelism": par, "compile": compile_flag, **note,
                       "loss": "logits + F.cross_entropy under loss_parallel (cut_cross_entropy is not installable offline)"},
            "clocks": clocks,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in pool[0].values()),
                    "d2h_bytes_per_step": 4, "last_loss": losses[-1]},
        }), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
