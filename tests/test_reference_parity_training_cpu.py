"""Training steps against the reference's stack, rank for rank: the reference's model under FSDP2 (``fully_shard`` per
block and at the root, as its ``parallelize_llama`` does) with ``torch.optim.AdamW``, and this repository's trainer with
its flat-buffer sharding runtime, start from the same weights and see the same batches on gloo ranks; per-step losses
and the final weights must agree.  fp32 on both sides (CPU)."""
import copy
import os
import sys

import pytest
import torch

from test_parallel_cpu import ADAMW, _batches, _cfg, _close, _load_full, run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "maester")), reason="the reference is not installed")


def _rank(rank, world, batches, family="llama3"):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, REF)
    import maester.models  # noqa: F401
    import torch.nn.functional as F
    from maester.models import model_name_to_cls as ref_cls, models_config as ref_cfgs
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from maester_b200.trainer import Trainer

    tp = family == "llama3_tp"
    if tp:
        family = "llama3"
    if family == "gemma3":   # tied embedding / head, sandwich norms, local and global layers
        import test_reference_parity_cpu as parity
        parity._adjust_reference_for_cpu()
        args = parity._small_gemma(ref_cfgs)
        args.n_layers = 3
    else:
        args = copy.deepcopy(ref_cfgs["llama3"]["debugmodel"])
        args.vocab_size = 512
    torch.manual_seed(11)   # same seed on every rank: same weights
    ref = ref_cls[family].from_model_args(args)
    ref.init_weights()
    if family == "gemma3":
        ref.set_attention_backend("naive")
        layers = ref.model.layers
    else:
        layers = ref.layers.values()
    full = {k: v.detach().clone() for k, v in ref.state_dict().items() if not k.endswith("freqs_cis")}
    if tp:
        # the reference's tensor-parallel plan (DTensor styles: column / row parallel linears, sequence-parallel norms,
        # all-gather / reduce-scatter along the sequence) on a mesh of two gloo ranks
        from maester.parallelisms.parallelize_llama import apply_tp
        apply_tp(ref, init_device_mesh("cpu", (world,), mesh_dim_names=("tp",)), loss_parallel=False, enable_async_tp=False)
    else:
        mesh = init_device_mesh("cpu", (world,))
        for layer in layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(ref, mesh=mesh)
    kw = dict(ADAMW[0]["opt_cfg"])
    opt = torch.optim.AdamW(ref.parameters(), lr=kw["lr"], betas=kw["betas"], weight_decay=kw["weight_decay"], eps=kw["eps"])

    if family == "gemma3":
        import maester_b200.models as ours
        ours.models_config["gemma3"]["parity"] = parity._small_gemma(ours.models_config)
        ours.models_config["gemma3"]["parity"].n_layers = 3
        tr = Trainer(_cfg(model_name="gemma3", flavor="parity", data_parallel_shard_degree=world))
    elif tp:
        tr = Trainer(_cfg(flavor="debugmodel", data_parallel_shard_degree=1, tensor_parallel_degree=world))
    else:
        tr = Trainer(_cfg(flavor="debugmodel", data_parallel_shard_degree=world))
    _load_full(tr, full, tp=(world, rank) if tp else None)

    per = batches[0]["input_ids"].shape[0] // (1 if tp else world)
    ref_losses, our_losses = [], []
    for b in batches:
        mine = b if tp else {k: v[rank * per:(rank + 1) * per] for k, v in b.items()}   # TP ranks share the batch
        loss = F.cross_entropy(ref(mine["input_ids"]).float().flatten(0, 1), mine["labels"].flatten())
        loss.backward()
        opt.step()
        opt.zero_grad()
        ref_losses.append(loss.item())
        our_losses.append(tr.train_step(mine).item())
    assert our_losses == pytest.approx(ref_losses, abs=2e-5), (ref_losses, our_losses)
    want = {n: p.full_tensor().detach() for n, p in ref.named_parameters()}
    got = {sl.fqn: sl.param.data for u in tr.sharded.units for sl in u.slots}
    if tp:
        from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
        want = tp_slice_state_dict(want, world, rank)
    assert sorted(want) == sorted(got)
    for k in want:
        assert _close(got[k], want[k], tol=2e-4), (k, ((got[k] - want[k]).norm() / want[k].norm()).item())
    return ref_losses


@pytest.mark.parametrize("world,family", [(1, "llama3"), (2, "llama3"), (2, "gemma3"), (2, "llama3_tp")])
def test_training_steps_follow_the_reference_under_fsdp2(world, family):
    os.environ["TORCHDYNAMO_DISABLE"] = "1"   # inherited by the spawned ranks: no host compiler set-up for Inductor here
    try:
        res = run_ranks(world, _rank, _batches(4, 2 * world, 64, 512), family)
    finally:
        os.environ.pop("TORCHDYNAMO_DISABLE", None)
    assert all(len(r) == 4 for r in res)
    if world == 2:
        assert (res[0] == res[1]) == (family == "llama3_tp")   # data-parallel ranks see different data
