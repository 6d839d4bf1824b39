"""Package-local resources (reference: npu_sparse_attn_sharedkv_int8/_paths.py:4-15)."""
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parent
NATIVE_DIR = PACKAGE_ROOT / "_native"
SCALES_PATH = PACKAGE_ROOT / "data" / "scales_v1.pt"
LIBRARY_NAME = "libsharedkv_cuda.so"


def native_path(filename=LIBRARY_NAME):
    path = NATIVE_DIR / filename
    if not path.is_file():
        raise RuntimeError(
            f"Missing native library {filename}. Build it with csrc/build.sh (nvcc, sm_100a); "
            "there is no CPU or framework fallback for the attention and cache-write kernels."
        )
    return path
