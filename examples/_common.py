"""Shared by the small examples: repository root on sys.path, the --device flag, and backend construction."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def parser(doc: str) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=doc, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cpu", help="cpu, or cuda:N for the B200 backend")
    ap.add_argument("--seed", type=int, default=0)
    return ap


def backend_for(device: str):
    from rustral_b200.core import B200Backend, CpuBackend
    return CpuBackend() if device == "cpu" else B200Backend(device)
