"""Regenerates the golden fixtures in this directory.  Run from the repository root, in a
container where the reference checkout is mounted:

    python tests/golden/make_golden.py --reference /path/to/NvFuserExamples

What it stores (all small, all produced by code that is NOT this repository's):
  ref_inference.npz  outputs of the reference's own `reference_mha` of test.py:12-18, whose
                     source is read from the checkout and executed on the CPU on seeded inputs
  ref_train.npz      same for `reference_mha` of test_train_mha.py:14-21 (softmax, dropout_out, ctx)
  philox_kat.npz     Philox4x32-10 outputs of PyTorch's host engine (oracle/philox_check.cpp)
The reference scripts cannot be imported as modules (they need a CUDA device and the built
extension at import time), so only the function definitions are extracted.
Inputs are regenerated from the stored seeds; a checksum of each input is stored to detect
a change of torch's CPU generator.
"""
from __future__ import annotations

import argparse
import ast
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def extract_function(path: Path, name: str, extra_globals: dict):
    tree = ast.parse(path.read_text())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            ns = dict(extra_globals)
            exec(compile(mod, str(path), "exec"), ns)
            return ns[name]
    raise KeyError(name)


def inference_inputs(seed: int, bh: int, s: int, d: int):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(bh, s, d, generator=g).to(torch.half)
    k = torch.randn(bh, s, d, generator=g).to(torch.half)
    v = torch.randn(bh, s, d, generator=g).to(torch.half)
    amask = torch.randint(0, 2, (bh, s, s), generator=g).to(torch.half)
    return q, k, v, amask


def train_inputs(seed: int, bh: int, s: int, d: int):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(bh, s, d, generator=g).to(torch.half)
    k = torch.randn(bh, s, d, generator=g).to(torch.half)
    v = torch.randn(bh, s, d, generator=g).to(torch.half)
    pad = torch.randint(0, 2, (bh, s, s), generator=g).to(torch.half) * (-1000)
    dm = torch.randint(0, 2, (bh, s, s), generator=g).to(torch.half)
    return q, k, v, pad, dm


def checksum(*tensors) -> np.ndarray:
    return np.array([float(t.double().sum()) for t in tensors])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of shmsong/NvFuserExamples")
    ns = ap.parse_args()
    ref = Path(ns.reference)

    # --- reference composites, executed as they are written -------------------------------
    f_inf = extract_function(ref / "test.py", "reference_mha", {"torch": torch})
    seed, bh, s, d = 11, 4, 128, 64
    q, k, v, amask = inference_inputs(seed, bh, s, d)
    ctx = f_inf(q, k, v, amask)
    np.savez_compressed(HERE / "ref_inference.npz", seed=seed, shape=np.array([bh, s, d]), ctx=ctx.numpy(),
                        input_checksum=checksum(q, k, v, amask))

    f_tr = extract_function(ref / "test_train_mha.py", "reference_mha",
                            {"torch": torch, "scale": 1.0 / 8, "dropout_prob": 0.5})
    seed, bh, s, d = 12, 2, 128, 64
    q, k, v, pad, dm = train_inputs(seed, bh, s, d)
    sm, dr, ctx = f_tr(q, k, v, pad, dm)
    np.savez_compressed(HERE / "ref_train.npz", seed=seed, shape=np.array([bh, s, d]), softmax=sm.numpy(),
                        dropout_out=dr.numpy(), ctx=ctx.numpy(), input_checksum=checksum(q, k, v, pad, dm))

    # --- Philox known answers from PyTorch's host engine -------------------------------------
    import torch.utils.cpp_extension as ce
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "_build/philox_check", f"TORCH_INCLUDE={ce.include_paths()[0]}"],
                   check=True, stdout=subprocess.DEVNULL)
    rng = np.random.default_rng(5)
    seeds = np.concatenate([np.array([0, 1, 2**64 - 1, 0x5EED0001], dtype=np.uint64), rng.integers(0, 2**63, 60, dtype=np.uint64)])
    ctrs = rng.integers(0, 2**32, (seeds.size, 4), dtype=np.uint64).astype(np.uint32)
    ctrs[0] = 0
    ctrs[2] = 0xFFFFFFFF
    text = "".join(f"{int(sd)} {int(c[0])} {int(c[1])} {int(c[2])} {int(c[3])}\n" for sd, c in zip(seeds, ctrs))
    out = subprocess.run([str(ROOT / "oracle" / "_build" / "philox_check")], input=text, capture_output=True, text=True,
                         check=True).stdout
    words = np.array([[int(x) for x in line.split()] for line in out.strip().splitlines()], dtype=np.uint32)
    assert words.shape == (seeds.size, 4)
    np.savez_compressed(HERE / "philox_kat.npz", seeds=seeds, counters=ctrs, words=words)
    print("wrote", [p.name for p in HERE.glob("*.npz")])


if __name__ == "__main__":
    sys.exit(main())
