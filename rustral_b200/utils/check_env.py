"""Environment check for building and running the framework (scripts/check_cuda_env.sh): toolkit version, the
in-tree libraries, the GPUs and their peer-access matrix.  Reads settings only; changes none.

    python -m rustral_b200.utils.check_env            # exit code 1 when something required is missing
    python -m rustral_b200.utils.check_env --json
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import subprocess
import sys

MIN_CUDA = (12, 8)          # first toolkit whose ptxas accepts sm_100a with the tcgen05 instructions used here


def parse_nvcc_version(text: str):
    m = re.findall(r"release (\d+)\.(\d+)", text)
    return (int(m[-1][0]), int(m[-1][1])) if m else None


def collect(run=subprocess.run) -> dict:
    info = {"problems": [], "warnings": []}
    nvcc = shutil.which("nvcc") or (os.path.exists("/usr/local/cuda/bin/nvcc") and "/usr/local/cuda/bin/nvcc") or None
    info["nvcc"] = nvcc
    if nvcc:
        try:
            out = run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
        except (OSError, subprocess.SubprocessError):
            out = ""
        ver = parse_nvcc_version(out)
        info["cuda_toolkit"] = list(ver) if ver else None
        if ver is None:
            info["problems"].append("could not parse the nvcc version")
        elif ver < MIN_CUDA:
            info["problems"].append(f"CUDA toolkit too old: nvcc reports {ver[0]}.{ver[1]}, need >= {MIN_CUDA[0]}.{MIN_CUDA[1]} "
                                    "for sm_100a")
    else:
        info["warnings"].append("nvcc not found: the in-tree libraries cannot be rebuilt here")
    import torch
    info["torch"] = torch.__version__
    info["torch_cuda"] = torch.version.cuda
    lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_lib")
    libs = {n: os.path.exists(os.path.join(lib_dir, n)) for n in ("librb200_kernels.so", "librb200_cpu.so", "librb200_runtime.so")}
    info["libraries"] = libs
    for n, ok in libs.items():
        if not ok:
            info["problems"].append(f"{n} is not built: run `python -m rustral_b200._build`")
    info["distributed_backends"] = {"nccl": bool(torch.distributed.is_available() and torch.distributed.is_nccl_available()),
                                    "gloo": bool(torch.distributed.is_available() and torch.distributed.is_gloo_available())}
    gpus = []
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                         "memory_gib": round(p.total_memory / 2 ** 30, 1)})
            if (p.major, p.minor) != (10, 0):
                info["problems"].append(f"GPU {i} ({p.name}) is sm_{p.major}{p.minor}; the kernels are built for sm_100a only")
        info["peer_access"] = [[i == j or bool(torch.cuda.can_device_access_peer(i, j)) for j in range(n)] for i in range(n)]
        if n > 1 and not all(all(r) for r in info["peer_access"]):
            info["warnings"].append("not every GPU pair has peer access: the fused multi-GPU paths need it")
    else:
        info["warnings"].append("no GPU visible: only the CPU reference backend and the build can be used")
    info["gpus"] = gpus
    info["ok"] = not info["problems"]
    return info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rustral_b200.utils.check_env")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    info = collect()
    if a.json:
        print(json.dumps(info, indent=1))
    else:
        tk = info.get("cuda_toolkit")
        print(f"nvcc: {info['nvcc'] or 'not found'}" + (f" (CUDA {tk[0]}.{tk[1]})" if tk else ""))
        print(f"torch {info['torch']} (CUDA {info['torch_cuda']}); backends: " +
              ", ".join(k for k, v in info["distributed_backends"].items() if v))
        print("libraries: " + ", ".join(f"{k}={'ok' if v else 'MISSING'}" for k, v in info["libraries"].items()))
        for g in info["gpus"]:
            print(f"GPU {g['index']}: {g['name']} sm_{g['sm']} {g['sms']} SMs {g['memory_gib']} GiB")
        for w in info["warnings"]:
            print("warning:", w)
        for p in info["problems"]:
            print("PROBLEM:", p)
        print("OK" if info["ok"] else "NOT OK")
    return 0 if info["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
