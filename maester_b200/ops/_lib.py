"""Build and load the native kernel library (``maester_b200/_C/libmaester_b200.so``).

The kernels are plain ``extern "C"`` launchers that take raw device pointers and a stream, so the
library has no dependency on torch headers: it compiles in seconds with a bare ``nvcc -shared`` and
is bound through ``ctypes``.  The shared object is built in-tree so that it travels with the
source tree to GPU machines.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent
CSRC = _PKG / "csrc"
OUT_DIR = _PKG / "_C"
# MB_CHECKED_KERNELS=1 selects the checked build (index checks in front of the kernels' global stores: a failing check
# skips the store and records a status code; see csrc/sm100.cuh::MB_CHECK_OR).  It is a separate shared object.
CHECKED = os.environ.get("MB_CHECKED_KERNELS", "0") == "1"
LIB_PATH = OUT_DIR / ("libmaester_b200_checked.so" if CHECKED else "libmaester_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]

_lib = None


def _nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > t for p in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link them into one shared object."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build maester_b200 kernels")
    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = OUT_DIR / ("obj_checked" if CHECKED else "obj")
    obj_dir.mkdir(exist_ok=True)
    procs = []
    objs = []
    hdr_t = max([p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))] or [0])
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_t):
            continue
        cmd = [nvcc, *NVCC_FLAGS, *(["-DMB_CHECKED"] if CHECKED else []), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
        if verbose and out:
            print(out)
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load the kernel library; raises if it is missing (a GPU run must never fall back silently)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            if _nvcc() is not None:
                build()
            else:
                raise RuntimeError(
                    f"{LIB_PATH} is missing and nvcc is unavailable: build it with "
                    "`python -c 'import __graft_entry__ as g; g.build()'`"
                )
        _lib = ctypes.CDLL(str(LIB_PATH))
        _declare(_lib)
    return _lib


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float


def _declare(l: ctypes.CDLL) -> None:
    sig = {
        "mb_gemm_bf16": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _L, _I, _I, _I, _F, _F, _P, _P],
        "mb_rmsnorm_fwd": [_P, _P, _P, _P, _P, _I, _I, _F, _I, _P],
        "mb_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
        "mb_qknorm_rope_fwd": [_P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _I, _L, _L, _P],
        "mb_qknorm_rope_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _I, _L, _L, _P],
        "mb_gemm_bf16_2cta": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _L, _I, _I, _I, _F, _F, _P, _P],
        "mb_gemm_bf16_grouped_rows": [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _I, _F, _P],
        "mb_gemm_bf16_grouped_contr": [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _F, _P],
        "mb_gemm_bf16_2cta_grouped_contr": [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _F, _P],
        "mb_fused_rs_adamw_ag": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _F, _F, _F, _F, _F, _F, _P],
        "mb_push_shards": [_P, _P, _P, _I, _P, _I, _P],
        "mb_peer_scatter_rows": [_P, _P, _I, _P, _P, _I, _I, _L, _P, _P],
        "mb_peer_gather_rows": [_P, _P, _I, _P, _P, _I, _I, _L, _P, _P],
        "mb_mla_pack_fwd": [_P, _P, _P, _L, _P, _P, _L, _I, _I, _I, _I, _I, _P, _P],
        "mb_mla_pack_bwd": [_P, _P, _P, _L, _I, _I, _I, _I, _I, _P, _P, _P, _P],
        "mb_ep_plan": [_P, _I, _I, _I, _I, _P, _P, _I, _I, _L, _P, _P, _P, _P],
        "mb_ep_zero_padding": [_P, _P, _I, _I, _I, _I, _P, _I, _L, _P],
        "mb_peer_dispatch_rows": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _L, _P, _P],
        "mb_peer_combine_rows": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _L, _P, _P],
        "mb_peer_slot_dot": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _L, _P],
        "mb_gemm_bf16_rs": [_P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _L, _I, _I, _F, _P],
        "mb_gemm_bf16_ag": [_P, _P, _I, _I, _P, _P, _I, _I, _I, _L, _L, _I, _I, _P, _P],
        "mb_gemm_bf16_ag_glu": [_P, _P, _I, _I, _P, _P, _I, _I, _I, _L, _L, _I, _P, _I, _I, _P, _L, _P],
        "mb_sum_partials": [_P, _P, _P, _L, _I, _P],
        "mb_pull_sum": [_P, _I, _I, _P, _P, _L, _L, _P],
        "mb_wait_flag_probe": [_P, _I, _F, _P, _P],
        "mb_symm_barrier": [_P, _I, _I, _I, _I, _F, _P],
        "mb_moe_route": [_P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _L] + [_P] * 15,
        "mb_moe_route_bwd": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
        "mb_moe_rows_gather": [_P, _P, _P, _I, _L, _I, _P, _P],
        "mb_moe_rows_combine": [_P, _P, _P, _I, _I, _I, _L, _P, _P],
        "mb_moe_slot_dot": [_P, _P, _P, _I, _I, _I, _L, _P, _P],
        "mb_syrk_bf16": [_P, _P, _P, _I, _I, _L, _L, _L, _F, _F, _P],
        "mb_gemm_glu_fwd": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _L, _I, _P],
        "mb_gemm_glu_bwd": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _L, _I, _P],
        "mb_glu_fwd": [_P, _P, _L, _I, _I, _L, _P],
        "mb_glu_bwd": [_P, _P, _P, _L, _I, _I, _L, _P],
        "mb_embedding_fwd": [_P, _P, _P, _L, _I, _F, _I, _P],
        "mb_embedding_bwd": [_P, _P, _P, _L, _I, _F, _P],
        "mb_ce_fwd_bwd": [_P, _P, _P, _P, _F, _L, _I, _L, _I, _I, _P, _P],
        "mb_set_norm_pipeline": [_I],
        "mb_gemm_ce": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _L, _F, _L, _P],
        "mb_ce_merge": [_P, _P, _P, _I, _I, _L, _P],
        "mb_ce_grad": [_P, _P, _P, _I, _P, _P, _L, _I, _L, _L, _I, _I, _P],
        "mb_expect_scalar": [_P, _F, _P],
        "mb_adamw": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _F, _F, _F, _F, _F, _F, _I, _P],
        "mb_peer_copy": [_P, _P, _L, _P],
        "mb_peer_gather": [_P, _L, _P, _I, _P, _I, _I, _P],
        "mb_peer_add_bf16": [_P, _P, _L, _P],
        "mb_attn_merge": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
        "mb_multi_sqnorm": [_P, _P, _I, _P, _P, _P],
        "mb_cast_f32_bf16": [_P, _P, _L, _F, _P],
        "mb_attn_fwd": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _L, _I, _I, _F, _P],
        "mb_attn_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                        _L, _L, _L, _L, _I, _I, _F, _P],
    }
    for name, args in sig.items():
        if hasattr(l, name):
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = _I
    l.mb_status.restype = _I
    l.mb_status_clear.restype = None
