"""The models compute the reference's functions: the reference's own model classes (installed copy of the reference
package) and this repository's models get the same weights, by parameter name, and must give the same logits, loss and
parameter gradients in fp32 on CPU.  Together with the GPU golden tests (native bf16 kernels against this repository's
fp32 path) this ties the kernels to the reference's definition of every model family.

Each family runs in a child process because the reference needs a few process-wide adjustments to run without a GPU,
none of which changes its arithmetic: ``TORCHDYNAMO_DISABLE=1`` (``torch.compile`` becomes the eager function; there is
no host compiler set-up for Inductor here), block masks built on ``cpu`` instead of the hard-coded ``cuda``, the "naive"
attention backend the reference ships for tests, ``torch.histc`` on integer input through a float copy (the CPU kernel
has no integer form), the permutation indices from the reference's own CPU routine instead of its Triton kernel, and no
forced flash backend around ``scaled_dot_product_attention``.
"""
import copy
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "maester")), reason="the reference is not installed")

FAMILIES = ["gemma3", "gemma3_packed", "gemma3_scaled", "llama3", "llama3_tied", "llama3_mup", "mistral", "glm4",
            "glm4_qknorm_bias", "deepseek", "deepseek_qlora_yarn"]


def _adjust_reference_for_cpu():
    import contextlib

    import torch
    import maester.models.deepseek.attention as ref_ds_attention
    import maester.models.gemma.model as ref_gemma
    import maester.models.moe.utils as ref_moe_utils

    make_mask = ref_gemma.create_block_mask
    ref_gemma.create_block_mask = lambda *a, **k: make_mask(*a, **{**k, "device": "cpu"})
    histc = torch.histc
    torch.histc = lambda x, *a, **k: histc(x, *a, **k) if x.is_floating_point() else histc(x.float(), *a, **k).to(x.dtype)
    indices = ref_moe_utils.generate_permute_indices
    ref_moe_utils.generate_permute_indices = lambda *a, **k: indices(*a, **{**k, "use_cpu": True})
    ref_ds_attention.sdpa_kernel = lambda *a, **k: contextlib.nullcontext()


def _small_gemma(cfgs):
    a = copy.deepcopy(cfgs["gemma3"]["270M"])
    for k, v in dict(vocab_size=512, dim=128, n_layers=7, n_heads=4, num_key_value_heads=2, head_dim=32,
                     intermediate_size=256, max_seq_len=128, sliding_window_size=16).items():
        setattr(a, k, v)   # 7 layers: the 5 local : 1 global pattern wraps; window 16 < sequence
    return a


def _pair(name, family, ref_cfgs, our_cfgs):
    import torch
    from maester.models import model_name_to_cls as ref_cls
    from maester_b200.models import model_name_to_cls as our_cls
    if name == "gemma3":
        ra, oa = _small_gemma(ref_cfgs), _small_gemma(our_cfgs)
        if family == "gemma3_scaled":   # what the 4B+ / 27B flavors add: scaled global RoPE, an explicit softmax scale
            for a in (ra, oa):
                a.rope_scaling, a.query_pre_attn_scalar = {"factor": 8.0}, 24
    else:
        flavor = {"llama3": "debugmodel", "llama3_tied": "tiny", "llama3_mup": "debugmodel", "mistral": "debugmodel",
                  "glm4": "debug", "glm4_qknorm_bias": "debug", "deepseek": "debug", "deepseek_qlora_yarn": "debug"}[family]
        ra, oa = copy.deepcopy(ref_cfgs[name][flavor]), copy.deepcopy(our_cfgs[name][flavor])
        ra.vocab_size = oa.vocab_size = 512
        if name == "deepseek":
            ra.max_seq_len = oa.max_seq_len = 96   # the reference applies its whole RoPE table: length == sequence
        for a in (ra, oa):
            if family == "llama3_mup":          # 1/d attention scale, output multiplier
                a.enable_mup, a.mup_width_mul, a.mup_output_alpha = True, 4.0, 2.0
            if family == "glm4_qknorm_bias":
                a.use_qk_norm, a.attention_bias = True, True
            if family == "deepseek_qlora_yarn":  # low-rank queries; sequence beyond the original length: YaRN + mscale
                a.q_lora_rank, a.original_seq_len, a.n_layers = 64, 32, 3
    torch.manual_seed(0)
    ref = ref_cls[name].from_model_args(ra)
    ref.init_weights()
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():   # norm weights off their initial value, so that their placement matters
        for n, p in ref.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn(p.shape, generator=g))
    if name == "gemma3":
        ref.set_attention_backend("naive")
    ours = our_cls[name].from_model_args(oa)
    ours.init_weights()
    missing, unexpected = ours.load_state_dict(dict(ref.state_dict()), strict=False)
    assert not missing and not [k for k in unexpected if not k.endswith("freqs_cis")], (missing, unexpected)
    return ref, ours, ra, oa


def _child(family: str) -> None:
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))   # stand-ins for packages the reference imports
    sys.path.insert(0, REF)
    sys.path.insert(0, ROOT)
    import torch
    import torch.nn.functional as F
    _adjust_reference_for_cpu()
    from maester.models import models_config as ref_cfgs
    from maester_b200.models import models_config as our_cfgs
    name = family.split("_")[0]
    ref, ours, ref_args, our_args = _pair(name, family, ref_cfgs, our_cfgs)
    bf16_experts = name in ("glm4", "deepseek")   # the reference runs its experts in bf16 whatever the model's dtype
    tol = 2e-2 if bf16_experts else 2e-5
    gen = torch.Generator().manual_seed(1)
    tok = torch.randint(0, 512, (2, 96), generator=gen)
    labels = torch.randint(0, 512, (2, 96), generator=gen)
    labels[0, :7] = -100

    if family == "gemma3_packed":
        # two documents packed into one row with position_ids / document_ids against the reference on each document
        # alone (its naive backend cannot take document_ids itself: the dense-mask helper fails on their shape)
        pos = torch.cat([torch.arange(40), torch.arange(56)])[None].expand(2, 96).contiguous()
        doc = torch.cat([torch.zeros(40, dtype=torch.long), torch.ones(56, dtype=torch.long)])[None].expand(2, 96).contiguous()
        with torch.no_grad():
            got = ours(tok, position_ids=pos, document_ids=doc).float()
            want = torch.cat([ref(tok[:, :40]).float(), ref(tok[:, 40:]).float()], dim=1)
        err = (got - want).abs().max().item()
        assert err < tol * want.abs().max().item(), err
        print(f"{family}: packed-document logits max abs diff {err:.2e}")
        return

    # parameter count and FLOPs per token (they set the reported MFU)
    counts = ref_args.get_nparams_and_flops(ref, 96)
    assert counts == our_args.get_nparams_and_flops(ours, 96), (counts, our_args.get_nparams_and_flops(ours, 96))
    a = ref(tok).float()
    b = ours(tok).float()
    scale = a.abs().max().item()
    err = (a - b).abs().max().item()
    assert a.shape == b.shape and err < tol * scale, (family, err, scale)
    # loss through each model's own loss path where it has one, else cross-entropy of the logits (the trainer's form)
    want_loss = F.cross_entropy(a.flatten(0, 1), labels.flatten(), ignore_index=-100)
    got_loss = ours(tok, labels=labels)
    assert abs(want_loss.item() - got_loss.item()) < max(tol, 1e-5) * 5, (want_loss.item(), got_loss.item())
    want_loss.backward()
    got_loss.backward()
    grads = dict(ours.named_parameters())
    worst = ("", 0.0)
    for n, p in ref.named_parameters():
        q = grads[n]
        assert (p.grad is None) == (q.grad is None or not q.grad.any()), n
        if p.grad is None:
            continue
        rel = ((p.grad - q.grad).norm() / (p.grad.norm() + 1e-12)).item()
        worst = max(worst, (n, rel), key=lambda t: t[1])
        assert rel < (5e-2 if bf16_experts else 1e-4), (n, rel)
    print(f"{family}: {counts[0]:,} parameters, {counts[1]:,} FLOPs/token; logits max abs diff {err:.2e} (scale {scale:.2f}), loss {want_loss.item():.6f} vs "
          f"{got_loss.item():.6f}, worst gradient {worst[0]} rel {worst[1]:.2e}")


@pytest.mark.parametrize("family", FAMILIES)
def test_models_compute_the_reference_functions(family):
    r = subprocess.run([sys.executable, os.path.abspath(__file__), family], capture_output=True, text=True,
                       env=dict(os.environ, TORCHDYNAMO_DISABLE="1"), timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    print(r.stdout.strip().splitlines()[-1])


if __name__ == "__main__":
    _child(sys.argv[1])
