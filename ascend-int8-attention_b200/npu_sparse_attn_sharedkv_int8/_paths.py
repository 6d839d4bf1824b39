"""Where the package keeps what is not Python (reference: npu_sparse_attn_sharedkv_int8/_paths.py:4-15)."""
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parent
NATIVE_DIR = PACKAGE_ROOT / "_native"                       # csrc/build.sh writes the library here
SCALES_PATH = PACKAGE_ROOT / "data" / "scales_v1.pt"        # where a deployment may place its frozen scales
LIBRARY_NAME = "libsharedkv_cuda.so"


def native_path(filename=LIBRARY_NAME):
    """Path of a built native artefact; RuntimeError when it has not been built."""
    candidate = NATIVE_DIR / filename
    if candidate.is_file():
        return candidate
    raise RuntimeError(f"Missing native library {filename}. Build it with csrc/build.sh (nvcc, sm_100a); "
                       "there is no CPU or framework fallback for the attention and cache-write kernels.")
