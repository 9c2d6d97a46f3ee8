"""Install the unmodified reference under baseline/_ref and prebuild its JIT CUDA extension for sm_100a (no GPU needed).

    python baseline/build_reference.py <path to the reference checkout>

1. `pip install --no-index --no-build-isolation --no-deps --target baseline/_ref` from a temporary copy of the checkout (the build
   writes into the source tree; torch is not in the offline wheelhouse, hence --no-deps).
2. Import the installed package with TORCH_CUDA_ARCH_LIST=10.0a and TORCH_EXTENSIONS_DIR=baseline/_ref/_torch_ext so that
   `gaac.kernel._ext()` and `gaac.vllm.paged_kernel._ext()` compile `gaac_attn_v1` and `gaac_vpaged128_v1` there (about three
   minutes each).  The directory string used for the build is
   recorded in baseline/_ref/_torch_ext/BUILD_DIR: ninja rebuilds when the paths in its command lines change, so
   run_reference_kernel.py reuses exactly that string when it still names the same directory.
Both outputs are git-ignored; they travel with the working tree to the GPU box.
"""
import os, shutil, subprocess, sys, tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def main():
    src = sys.argv[1]
    if not os.path.isdir(os.path.join(REF, "gaac")):
        with tempfile.TemporaryDirectory() as tmp:
            cp = os.path.join(tmp, "reference")
            shutil.copytree(src, cp)
            subprocess.check_call([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                                   "--find-links", "/opt/wheelhouse", "--target", REF, cp])
    ext = os.path.join(REF, "_torch_ext")
    os.makedirs(ext, exist_ok=True)
    env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0a", TORCH_EXTENSIONS_DIR=ext, MAX_JOBS=str(os.cpu_count() or 4))
    subprocess.check_call([sys.executable, "-c", f"import sys; sys.path.insert(0, {REF!r}); from gaac import kernel; print(kernel._ext()); "
                           "from gaac.vllm import paged_kernel; print(paged_kernel._ext())"], env=env)
    with open(os.path.join(ext, "BUILD_DIR"), "w") as f:
        f.write(ext)
    print("reference installed under", REF, "; extension prebuilt under", ext)


if __name__ == "__main__":
    main()
