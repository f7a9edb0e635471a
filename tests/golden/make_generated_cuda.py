"""Copies the `## CUDA C` blocks of the reference's generated-code files into tests/golden/generated_cuda/.

The reference keeps, for every benchmark kernel, the source text its backends generate from the kernel's IR
(benchmarks/descriptions/generated/<name>_generated.md); its CI regenerates these files and fails when they
differ (.github/workflows/ci.yml:150-184), so they are golden renderings of the real IR that the PPX lowers.
The blocks for the kernels on this backend's path are stored one per file, byte for byte, as fixtures for
tests/test_ir_golden.py.  Needs the reference tree; run once where it is mounted:

    python tests/golden/make_generated_cuda.py /path/to/reference
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
KERNELS = ["matrix_mul", "matrix_mul_tiled", "vector_add", "stream_triad", "dot_product", "reduction", "vector_copy"]


def cuda_block(md_text: str) -> str:
    start = md_text.index("## CUDA C")
    fence = md_text.index("```cuda\n", start) + len("```cuda\n")
    end = md_text.index("```", fence)
    return md_text[fence:end]


def main(ref_root: str) -> None:
    out_dir = os.path.join(HERE, "generated_cuda")
    os.makedirs(out_dir, exist_ok=True)
    for name in KERNELS:
        with open(os.path.join(ref_root, "benchmarks", "descriptions", "generated", name + "_generated.md")) as f:
            block = cuda_block(f.read())
        with open(os.path.join(out_dir, name + ".cu.txt"), "w") as f:
            f.write(block)
        print(name, len(block), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_generated_cuda.py /path/to/reference")
    main(sys.argv[1])
