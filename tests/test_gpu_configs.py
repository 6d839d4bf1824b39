"""The benchmark configurations at their stated geometry, on the GPU, against the oracle.

Configuration 1: a C128 layer, 64 requests, one query token each, contexts uniform over
8 192..131 072 tokens, compact pages (38 slots of 16 384 bytes per block = a 622 592-byte page
stride, payload one slot in).  Configuration 2: a C4 layer with one speculative token (T = 2),
256 requests, contexts uniform over 32 768..131 072, top-k 1024 per query token.  The launches are
the ones `bench.py --workload c128 / c4mtp` times.  Sampled requests are extracted as small CPU
cases and compared with the oracle twice: inside the acceptance band against one running state per
token (max-abs 2e-2, mean-abs 2e-3), and inside the reference's own device band (rtol 0.008,
atol 0.0003, LSE 2e-5; tests/npu/test_attention.py:102-103 of the reference) against the oracle
dealt the same tile pieces as the launch.
"""
from types import SimpleNamespace

import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import device_tile_parts, error_metrics

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"
SAMPLED = 20


def run_and_compare(work, layer_index=0, sampled=SAMPLED):
    from npu_sparse_attn_sharedkv_int8 import synthetic
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    layer = work.layers[layer_index]
    op = PreparedAttention(work.case(layer_index), layer.ori_scale, layer.cmp_scale, return_lse=True)
    out, lse = op.run().clone(), op.lse.clone()
    torch.cuda.synchronize()
    assert torch.equal(op.run(), out)                                  # repeat launches give the same bits
    c8 = __import__("npu_sparse_attn_sharedkv_int8.c8_attention", fromlist=["workspace_status"])
    c8.workspace_status(op)                                            # no wait inside the kernel ran out

    # shortest, longest and a spread of the requests in between
    order = torch.argsort(work.seq_lens_host).tolist()
    step = max(1, len(order) // (sampled - 2))
    sample = sorted(set(order[::step][:sampled - 2]) | {order[0], order[-1]})
    assert len(sample) >= min(16, sampled - 2, len(order))
    small, ori_scale, cmp_scale, ids = synthetic.extract_requests(work, layer_index, sample)
    got, got_lse = out[ids.to(DEVICE)].cpu().float(), lse[ids.to(DEVICE)].cpu()

    expected, expected_lse = oracle.attention_tiled(small, ori_scale, cmp_scale, return_lse=True)
    m = error_metrics(got, expected.float())
    assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
    torch.testing.assert_close(got_lse, expected_lse, rtol=1e-4, atol=1e-4)

    # the same tile pieces as the launch: the split of the whole batch, looked up for the sampled tokens
    whole = SimpleNamespace(seq_lens=work.seq_lens_host, cu_q=torch.arange(0, work.tokens + 1, work.queries),
                            ratio=layer.ratio, cmp_indices=layer.cmp_indices)
    ctas = min(torch.cuda.get_device_properties(0).multi_processor_count, 160)
    parts = device_tile_parts(whole, ctas)
    dealt = {}
    for new, old in enumerate(ids.tolist()):
        first = min(parts[old])
        dealt[new] = [p - first for p in parts[old]]
    expected, expected_lse = oracle.attention_tiled(small, ori_scale, cmp_scale, return_lse=True, tile_parts=dealt)
    torch.testing.assert_close(got, expected.float(), rtol=0.008, atol=0.0003)
    torch.testing.assert_close(got_lse, expected_lse, rtol=2e-5, atol=2e-5)
    return m


def test_config1_c128_compact_pages():
    from npu_sparse_attn_sharedkv_int8 import synthetic
    lengths = synthetic.uniform_lengths(64, 8192, 131072, seed=1)
    work = synthetic.build("c128", DEVICE, lengths, ratios=[128], queries=1, seed=200, stride_slots=38, slot_offset=1,
                           max_context=135000)
    layer = work.layers[0]
    assert layer.cmp.stride(0) == 622592 and layer.ori.stride(0) == 622592
    assert (layer.cmp.data_ptr() - work.pools[1].data_ptr()) == 16384          # payload one slot into the block
    run_and_compare(work)
    del work
    torch.cuda.empty_cache()


def test_config2_c4_with_a_speculative_token():
    from npu_sparse_attn_sharedkv_int8 import synthetic
    lengths = synthetic.uniform_lengths(256, 32768, 131072, seed=2)
    work = synthetic.build("c4mtp", DEVICE, lengths, ratios=[4], queries=2, seed=300, max_context=135000)
    assert work.tokens == 512 and work.layers[0].cmp_indices.shape == (512, 1, 1024)
    run_and_compare(work)
    del work
    torch.cuda.empty_cache()
