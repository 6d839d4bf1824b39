"""Batch and context capacities the reference runs on its device (tests/npu/test_capacity.py:30-60 of the
reference: batches of 9 to 512 requests, one or six query tokens each, contexts of 129 to 65 536
tokens, both layer kinds), at their geometry on the GPU.  A handful of requests of every launch is
extracted and walked by the oracle: acceptance band against one running state per token, and the
reference's device band against the oracle dealt the tile pieces of the launch."""
import pytest
import torch

from tests.test_gpu_configs import run_and_compare

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"

SHAPES = [(23, 6, 8192), (32, 1, 32768), (32, 6, 65536), (64, 1, 8192), (64, 6, 8192), (128, 1, 4096), (128, 6, 4096),
          (256, 1, 513), (9, 1, 129), (23, 1, 8193), (48, 1, 1028), (49, 1, 1028), (512, 1, 129)]


@pytest.mark.parametrize("ratio", (4, 128))
@pytest.mark.parametrize("batch,queries,length", SHAPES)
def test_capacity_shape(ratio, batch, queries, length):
    from npu_sparse_attn_sharedkv_int8 import synthetic
    lengths = torch.full((batch,), length, dtype=torch.int64)
    work = synthetic.build("capacity", DEVICE, lengths, ratios=[ratio], queries=queries, seed=batch * 7 + queries, max_context=length + 64)
    run_and_compare(work, sampled=8)
    del work
    torch.cuda.empty_cache()
