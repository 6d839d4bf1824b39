#!/bin/sh
# Builds libsharedkv_cuda.so for sm_100a into the Python package's _native directory.
set -e
here=$(cd -- "$(dirname -- "$0")" && pwd)
out="$here/../npu_sparse_attn_sharedkv_int8/_native"
mkdir -p "$out"
NVCC=${NVCC:-/usr/local/cuda/bin/nvcc}
"$NVCC" -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a \
    -Xcompiler -fPIC -Xcompiler -fvisibility=hidden \
    -shared -o "$out/libsharedkv_cuda.so" \
    "$here/c_abi.cu" "$here/cache_write.cu" "$here/decode_attention.cu" \
    "$here/attention_static_scratch.cu"
echo "built $out/libsharedkv_cuda.so"
