"""Generates the golden vectors under tests/golden/ from the REFERENCE's own kernels.

Run on a machine with a CUDA GPU after `make -C oracle` has compiled the reference kernels
unchanged into oracle/_ref (naive/naive_1.cu, shared/shared_2.cu, blocktile_1d/blocktile_1d.cu):

    python tests/golden/make_golden.py [output_dir]

For every case the three reference kernels are run on the same seeded inputs; they must agree
bit for bit with each other (they do: same accumulation order), and that common output is stored
with the seed and shape.  Inputs are regenerated from the seed by the tests
(oracle.gen_randn_f32 / gen_uniform_f32), so only C is stored.  Files are a few hundred KB.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

# (generator, seed, M, K, N)
CASES = [
    ("randn", 42, 128, 128, 128),      # the reference tests' first shape and seed (naive/test.py:13,17)
    ("randn", 42, 64, 300, 48),
    ("uniform", 0, 96, 1024, 80),      # long K: rounding-order sensitive
    ("uniform", 0, 33, 17, 65),        # ragged, exercises the reference's guards
    ("randn", 7, 200, 77, 130),
]


def main(out_dir: Path) -> None:
    assert torch.cuda.is_available() and O.reference_available()
    out_dir.mkdir(parents=True, exist_ok=True)
    for gen, seed, M, K, N in CASES:
        A, B = (O.gen_randn_f32 if gen == "randn" else O.gen_uniform_f32)(M, K, N, seed=seed)
        outs = []
        for v in ("naive", "shared", "blocktile_1d"):
            C = torch.zeros(M, N, device="cuda")
            outs.append(O.reference_kernel(v)(A.cuda(), B.cuda(), C).cpu())
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), "reference kernels disagree"
        name = f"ref_sgemm_{gen}{seed}_{M}x{K}x{N}.npz"
        np.savez_compressed(out_dir / name, C=outs[0].numpy(), gen=gen, seed=seed, M=M, K=K, N=N,
                            a_checksum=float(A.double().sum()), b_checksum=float(B.double().sum()))
        print("wrote", name)


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent)
