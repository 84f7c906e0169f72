#!/usr/bin/env python3
"""Copies the known-answer tensors that llmt's own tests hold for the matmul
path into tests/golden/llmt/ so the parity tests can run where the llmt source
tree is not present.

Source: <llmt>/tests/golden/{matmul,matmul_rank3,linear,mlp,attention,gelu,permute,cross_entropy}/*.bin
(written by llmt's tools/gen_golden.py with PyTorch on CPU; asserted by
tests/unit/test_matmul.cu, test_linear.cu, test_mlp.cu, test_attention.cu and
test_kernels_fwd.cu at rtol 1e-5 / atol 1e-6; the permute case at 1e-6 / 1e-7; cross_entropy
(the consumer of the LM-head logits) by test_cross_entropy.cu at 1e-5 / 1e-6).

The files are data, copied byte for byte. Usage:
    python tests/golden/import_llmt_goldens.py <path-to-llmt-tree>
"""
import os
import shutil
import sys

CASES = ["matmul", "matmul_rank3", "linear", "mlp", "attention", "gelu", "permute", "cross_entropy"]


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    src_root = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    for case in CASES:
        src = os.path.join(src_root, "tests", "golden", case)
        dst = os.path.join(here, "llmt", case)
        os.makedirs(dst, exist_ok=True)
        for name in sorted(os.listdir(src)):
            if name.endswith(".bin"):
                shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
                print(f"{case}/{name}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
