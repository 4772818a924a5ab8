"""Post-install step (flextrain/scripts/post_install.py:1-28).

The reference uses this hook to download prebuilt flash-attn and causal-conv1d wheels.  This package carries its own
attention and convolution kernels, so nothing is fetched from the network; the hook builds the in-tree native
libraries and then checks the installation the way a first run would meet it:

* tool chain: ``nvcc`` present and able to target ``sm_100a``, a host C++ compiler;
* every native library builds, loads (``dlopen``) and exports its entry points;
* GPUs: compute capability 10.0 (the kernels are built for nothing else), peer access between every pair of
  devices of the node (the fused collectives read and write peers' memory), host memory the process may pin;
* optional packages used only as comparison bars (``flash_attn``, ``fla``) or by the comparison harness
  (``transformers``, ``torchtitan``).

Exit status 1 when something the training path needs is missing; missing optional items are listed and ignored.

    python -m flextrain_b200.scripts.post_install [--no-build] [--json]
"""
from __future__ import annotations

import argparse
import ctypes
import importlib.util
import json
import shutil
import subprocess
from typing import Dict, List

# one exported entry point per library: enough to tell a complete build from a truncated one
ENTRY_POINTS = {
    "gemm_tcgen05": "ftb_gemm_bf16", "elementwise": "ftb_adamw_multi", "attention": "ftb_attn_fwd",
    "comm": "ftb_comm_adamw_push", "moe": "ftb_ep_plan_count", "noalloc": "ftb_rmsnorm_bwd_noalloc",
    "gdn": "ftb_gdn", "seqmix": "ftb_conv1d_fwd", "dp_solver": "ftb_dp_solve", "copy_engine": "ftb_ce_create",
}
OPTIONAL = {"flash_attn": "attention comparison bar", "fla": "Gated DeltaNet comparison bar",
            "transformers": "HF parity tests and the hf_fsdp2 baseline", "torchtitan": "torchtitan baseline"}


def check_toolchain() -> Dict[str, object]:
    from ..build import NVCC
    out: Dict[str, object] = {"nvcc": None, "sm_100a": False, "cxx": shutil.which("g++")}
    if shutil.which(NVCC) or shutil.os.path.exists(NVCC):
        try:
            v = subprocess.run([NVCC, "--version"], capture_output=True, text=True, timeout=60).stdout
            out["nvcc"] = next((l.strip() for l in v.splitlines() if "release" in l), v.strip()[-80:])
            archs = subprocess.run([NVCC, "--list-gpu-code"], capture_output=True, text=True, timeout=60).stdout.split()
            out["sm_100a"] = "sm_100" in archs          # the listing names base architectures; "a" is a build flag
        except Exception as e:                             # a broken tool chain is a finding, not a crash
            out["error"] = f"{type(e).__name__}: {e}"
    return out


def check_libraries(build: bool = True) -> Dict[str, Dict[str, object]]:
    from ..build import LIB, build_all, lib_path
    res: Dict[str, Dict[str, object]] = {}
    if build:
        try:
            build_all()
        except RuntimeError as e:
            res["_build"] = {"ok": False, "error": str(e)[-400:]}
    for name, sym in ENTRY_POINTS.items():
        p = lib_path(name)
        r: Dict[str, object] = {"path": str(p), "ok": False}
        if not p.exists():
            r["error"] = "not built"
        else:
            try:
                lib = ctypes.CDLL(str(p))
                r["ok"] = hasattr(lib, sym)
                if not r["ok"]:
                    r["error"] = f"entry point {sym} is missing"
            except OSError as e:
                r["error"] = str(e)[:200]
        res[name] = r
    ext = sorted(LIB.glob("_ftb_fastcall*.so")) if LIB.exists() else []
    res["fastcall"] = {"path": str(ext[0]) if ext else None, "ok": bool(ext)}
    if not ext:
        res["fastcall"]["error"] = "not built"
    return res


def check_gpus() -> Dict[str, object]:
    import torch
    from ..core._memory import get_available_host_memory
    out: Dict[str, object] = {"available": torch.cuda.is_available(), "devices": [], "peer_access": None,
                              "host_memory_gib": round(get_available_host_memory() / 2 ** 30, 1)}
    if not out["available"]:
        return out
    n = torch.cuda.device_count()
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        out["devices"].append({"index": i, "name": p.name, "cc": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                               "memory_gib": round(p.total_memory / 2 ** 30), "supported": (p.major, p.minor) == (10, 0)})
    if n > 1:
        out["peer_access"] = all(torch.cuda.can_device_access_peer(a, b) for a in range(n) for b in range(n) if a != b)
    return out


def check_optional() -> Dict[str, bool]:
    return {m: importlib.util.find_spec(m) is not None for m in OPTIONAL}


def problems(report: dict) -> List[str]:
    """What keeps the training path from running, as sentences."""
    bad: List[str] = []
    tc, libs, gpus = report["toolchain"], report["libraries"], report["gpus"]
    missing = [n for n, r in libs.items() if not r.get("ok")]
    if missing:
        why = "" if tc.get("nvcc") and tc.get("sm_100a") else " (nvcc with sm_100a support is needed to build them)"
        bad.append("native libraries not usable: " + ", ".join(sorted(missing)) + why)
    for d in gpus["devices"]:
        if not d["supported"]:
            bad.append(f"cuda:{d['index']} is compute capability {d['cc']}; the kernels are built for 10.0 (sm_100a) only")
    if gpus["peer_access"] is False:
        bad.append("not every pair of GPUs has peer access; multi-GPU runs fall back to FTB_DP_BACKEND=collective")
    return bad


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--no-build", action="store_true", help="check what is there; compile nothing")
    ap.add_argument("--json", action="store_true", help="print the report as one JSON object")
    args = ap.parse_args(argv)
    report = {"toolchain": check_toolchain(), "libraries": check_libraries(build=not args.no_build),
              "gpus": check_gpus(), "optional": check_optional()}
    report["problems"] = problems(report)
    if args.json:
        print(json.dumps(report))
        return 1 if report["problems"] else 0
    tc = report["toolchain"]
    print(f"[post-install] nvcc: {tc['nvcc'] or 'not found'}; sm_100a target: {'yes' if tc['sm_100a'] else 'no'}; "
          f"g++: {tc['cxx'] or 'not found'}")
    for name, r in sorted(report["libraries"].items()):
        print(f"[post-install] {name}: " + (str(r["path"]) if r.get("ok") else f"MISSING ({r.get('error')})"))
    g = report["gpus"]
    if not g["available"]:
        print("[post-install] no GPU visible (the libraries still build; training needs a B200)")
    for d in g["devices"]:
        print(f"[post-install] cuda:{d['index']} {d['name']} cc {d['cc']} {d['memory_gib']} GiB {d['sms']} SMs"
              + ("" if d["supported"] else "  <- not sm_100"))
    if g["peer_access"] is not None:
        print(f"[post-install] peer access between all GPUs: {'yes' if g['peer_access'] else 'NO'}")
    print(f"[post-install] host memory available to this process: {g['host_memory_gib']} GiB")
    for m, ok in report["optional"].items():
        print(f"[post-install] optional {m}: {'found' if ok else 'absent'} ({OPTIONAL[m]})")
    for line in report["problems"]:
        print("[post-install] PROBLEM: " + line)
    return 1 if report["problems"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
