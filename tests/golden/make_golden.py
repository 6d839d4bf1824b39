"""Generate the golden vectors under tests/golden/ from the reference project itself.

Run once, in a container that has the reference checkout (it is not needed to run the
tests):

    TORCH_DEVICE_BACKEND_AUTOLOAD=0 python tests/golden/make_golden.py --reference /path/to/reference

Every array written here is an input to, or an output of, the reference's own Python
functions: `CacheQuantization.quantize`, `tiled_quantized_reference`, `sharedkv_reference`
and `joint_quantized_row` (npu_sparse_attn_sharedkv_int8/reference.py) and, for the
"real" cases, `ActivationCorpus.make` (tests/support/serving_shapes.py) with the frozen
scale file shipped in the reference package.  BF16 tensors are stored as their uint16 bit
patterns.  The tests compare the oracle in oracle/ and the CUDA library against them.
"""
import argparse
from dataclasses import replace
import math
from pathlib import Path
import sys

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def save_case(name, case, oq, cq, ref, extra=None):
    torch.set_num_threads(4)
    arrays = dict(
        q=bits(case.q), ori=case.ori.numpy(), ori_table=case.ori_block_table.numpy(),
        cmp=case.cmp.numpy(), cmp_table=case.cmp_block_table.numpy(),
        cu_q=case.cu_q.numpy(), seq_lens=case.seq_lens.numpy(), sink=case.sink.numpy(),
        ori_scale=oq.scale.numpy(), cmp_scale=cq.scale.numpy(),
        ratio=np.int32(case.ratio), softmax_scale=np.float64(case.softmax_scale))
    if case.cmp_indices is not None:
        arrays['cmp_indices'] = case.cmp_indices.numpy()
    for splits in (1, 2, 3):
        out, lse = ref.tiled_quantized_reference(case, oq, cq, tile_size=128, splits=splits, return_lse=True)
        arrays[f'out_s{splits}'] = bits(out)
        arrays[f'lse_s{splits}'] = lse.numpy()
    decoded = replace(case, ori=oq.dequantize(case.ori), cmp=cq.dequantize(case.cmp))
    out64, lse64 = ref.sharedkv_reference(decoded)
    arrays['out_fp64'] = out64.numpy()
    arrays['lse_fp64'] = lse64.numpy()
    if extra:
        arrays.update(extra)
    np.savez_compressed(HERE / f'{name}.npz', **arrays)
    print(name, {k: v.shape for k, v in arrays.items() if hasattr(v, 'shape') and v.ndim}, flush=True)


def windowed_case(ref, *, ratio, queries, lengths, seed, topk=1024, edit_indices=None):
    """Synthetic case of the benchmark configuration family: lognormal per-channel spread, scale =
    1.1 * absmax / 127, page tables that are random permutations of the page pool, and only
    the window pages of the original cache allocated (as a sliding-window allocator does)."""
    g = torch.Generator().manual_seed(seed)
    batch, tokens = len(queries), sum(queries)
    sigma = torch.exp(torch.randn(512, generator=g) * 0.5)

    def pool(ranges, width):
        count = max(1, sum(len(r) for r in ranges))
        order = torch.randperm(count, generator=g, dtype=torch.int32)
        table = torch.zeros((batch, width), dtype=torch.int32)
        offset = 0
        for b, r in enumerate(ranges):
            if len(r):
                table[b, list(r)] = order[offset:offset + len(r)]
                offset += len(r)
        rows = (torch.randn(count, 32, 1, 512, generator=g) * sigma).bfloat16()
        return rows, table

    ori_ranges = [range(max(0, s - q - 127) // 32, (s - 1) // 32 + 1) for q, s in zip(queries, lengths)]
    ori, ori_table = pool(ori_ranges, math.ceil(max(lengths) / 32))
    cmp_ranges = [range(math.ceil((s // ratio) / 32)) for s in lengths]
    cmp, cmp_table = pool(cmp_ranges, max(1, math.ceil(max(lengths) / (ratio * 32))))
    oq = ref.CacheQuantization((ori.float().reshape(-1, 512).abs().amax(0) * 1.1 / 127).clamp_min(1e-8))
    cq = ref.CacheQuantization((cmp.float().reshape(-1, 512).abs().amax(0) * 1.1 / 127).clamp_min(1e-8))
    indices = None
    if ratio == 4:
        indices = torch.full((tokens, 1, topk), -1, dtype=torch.int32)
        t = 0
        for q, s in zip(queries, lengths):
            for local in range(q):
                count = (s - q + local + 1) // 4
                chosen = torch.randperm(count, generator=g, dtype=torch.int32)[:topk]
                indices[t, 0, :len(chosen)] = chosen
                t += 1
        if edit_indices is not None:
            edit_indices(indices, g)
    cu = torch.tensor([0, *np.cumsum(queries).tolist()], dtype=torch.int32)
    case = ref.SharedKVCase(q=torch.randn(tokens, 8, 512, generator=g).bfloat16(), ori=oq.quantize(ori),
                            ori_block_table=ori_table, cu_q=cu, seq_lens=torch.tensor(lengths, dtype=torch.int32),
                            sink=torch.linspace(-2, 2, 8), cmp=cq.quantize(cmp), cmp_block_table=cmp_table,
                            cmp_indices=indices, ratio=ratio)
    return case, oq, cq


def layout_golden(reference):
    """cache_layout.json: offsets, strides and group splits computed by the reference's own
    `cache_layout.uses_compact / group_specs / packed_layout` (npu_sparse_attn_sharedkv_int8/
    cache_layout.py:24-85) on vLLM's real cache-spec objects.  Only that one file of the reference is
    loaded (by path: its package name is also this build's), and it imports nothing but vLLM."""
    import importlib.util
    import json
    from vllm.v1.kv_cache_interface import KVCacheGroupSpec, MLAAttentionSpec, UniformTypeKVCacheSpecs
    spec = importlib.util.spec_from_file_location('reference_cache_layout',
                                                  reference / 'npu_sparse_attn_sharedkv_int8' / 'cache_layout.py')
    layout = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(layout)

    def mla(dtype, head_size, block_size=32, padded=None, ratio=1, version='deepseek_v4'):
        return MLAAttentionSpec(block_size=block_size, num_kv_heads=1, head_size=head_size, dtype=dtype,
                                page_size_padded=padded, compress_ratio=ratio, model_version=version)

    def describe(name, s):
        return dict(name=name, dtype=str(s.dtype).replace('torch.', ''), page_size_bytes=s.page_size_bytes,
                    head_size=s.head_size, block_size=s.block_size, num_kv_heads=s.num_kv_heads,
                    page_size_padded=s.page_size_padded, model_version=getattr(s, 'model_version', None),
                    unpadded_page_size_bytes=replace(s, page_size_padded=None).page_size_bytes)

    def uniform(specs):
        merged = UniformTypeKVCacheSpecs.from_specs(specs)
        assert merged is not None
        return merged

    scenarios = {}
    # the serving geometry of the reference's device tests: 38 INT8 D=512 layers in one group
    # (38 x 16 384 = 622 592 bytes per block) beside a group of FP32 compressor states
    attention = {f'model.layers.{i}.attn': mla(torch.int8, 512) for i in range(38)}
    states = {f'model.layers.{i}.state': mla(torch.float32, 130, block_size=8) for i in range(6)}
    scenarios['serving38'] = [attention, states]
    # vLLM's own page sizes for compressed layers (a page holds block_size / compress_ratio rows)
    scenarios['compressed_pages'] = [{f'm.{i}.attn': mla(torch.int8, 512, ratio=4 if i % 2 == 0 else 128) for i in range(6)}]
    # mixed sizes inside a group: ordering by size and alignment
    scenarios['mixed'] = [{'a.small': mla(torch.int8, 100), 'a.big': mla(torch.int8, 512), 'a.mid': mla(torch.int8, 129)},
                          {'b.f32': mla(torch.float32, 65), 'b.big': mla(torch.int8, 512)}]
    # INT8 D=512 caches of another model version, and BF16 caches: not compact
    scenarios['other_model'] = [{'x.attn': mla(torch.int8, 512, version='deepseek_v3')}]
    scenarios['bf16'] = [{'y.attn': mla(torch.bfloat16, 512)}]
    result = {}
    for name, groups in scenarios.items():
        group_objects = [KVCacheGroupSpec(list(specs), uniform(specs)) for specs in groups]
        stride, offsets = layout.packed_layout(group_objects)
        result[name] = dict(groups=[[describe(n, s) for n, s in specs.items()] for specs in groups],
                            uses_compact=bool(layout.uses_compact(group_objects)), stride=stride, offsets=offsets,
                            pool_bytes_per_block=layout.pool_bytes_per_block(group_objects))
    # group_specs: C4 (cache + indexer), C128, and an over-full group of padded FP32 states
    c4 = {'l0.c4': mla(torch.int8, 512, ratio=4), 'l0.indexer': mla(torch.int8, 132, ratio=4)}
    c128 = {'l1.c128': mla(torch.int8, 512, ratio=128)}
    padded = {f'l{i}.state': mla(torch.float32, 128, padded=32768) for i in range(5)}
    grouped = [uniform(c4), uniform(c128), uniform(padded)]
    split = layout.group_specs(grouped)
    result['group_specs'] = dict(
        groups=[[describe(n, s) for n, s in specs.items()] for specs in (c4, c128, padded)],
        split=[[describe(n, g.kv_cache_spec.kv_cache_specs[n]) for n in g.layer_names] for g in split])
    (HERE / 'cache_layout.json').write_text(json.dumps(result, indent=1, sort_keys=True) + '\n')
    print('cache_layout', {k: v.get('stride') for k, v in result.items()}, flush=True)


def slots_golden(ref):
    """slots_swa.npz / slots_c4.npz: explicit original slots through the reference's tiled oracle."""
    # ---- explicit original slots (reference.py:235-239): a ratio-1 layer as the draft model's
    #      attention uses it (no compressed cache, 300 physical slots per token with holes, out-of-range
    #      entries and duplicates), and a C4 layer with 160 slots in place of the window
    def slot_case(ratio, queries, lengths, slots_per_token, seed):
        case, oq, cq = windowed_case(ref, ratio=max(ratio, 4), queries=queries, lengths=lengths, seed=seed)
        g = torch.Generator().manual_seed(seed + 100)
        total = case.ori.shape[0] * 32
        slots = torch.randint(0, total, (sum(queries), 1, slots_per_token), generator=g, dtype=torch.int32)
        slots[:, :, ::9] = -1
        slots[:, :, 4::17] = total + 5
        slots[0, 0, 10:20] = slots[0, 0, 30:40]
        if ratio == 1:
            case = replace(case, cmp=None, cmp_block_table=None, cmp_indices=None, ratio=1)
        return replace(case, ori_indices=slots), oq, cq

    def save_slot_case(name, case, oq, cq):
        arrays = dict(q=bits(case.q), ori=case.ori.numpy(), ori_table=case.ori_block_table.numpy(), cu_q=case.cu_q.numpy(),
                      seq_lens=case.seq_lens.numpy(), sink=case.sink.numpy(), ori_scale=oq.scale.numpy(),
                      ratio=np.int32(case.ratio), softmax_scale=np.float64(case.softmax_scale), ori_indices=case.ori_indices.numpy())
        if case.ratio != 1:
            arrays.update(cmp=case.cmp.numpy(), cmp_table=case.cmp_block_table.numpy(), cmp_scale=cq.scale.numpy(),
                          cmp_indices=case.cmp_indices.numpy())
        for splits in (1, 2):
            out, lse = ref.tiled_quantized_reference(case, oq, cq if case.ratio != 1 else None, tile_size=128, splits=splits,
                                                     return_lse=True)
            arrays[f'out_s{splits}'] = bits(out)
            arrays[f'lse_s{splits}'] = lse.numpy()
        np.savez_compressed(HERE / f'{name}.npz', **arrays)
        print(name, {k: v.shape for k, v in arrays.items() if hasattr(v, 'shape') and v.ndim}, flush=True)

    save_slot_case('slots_swa', *slot_case(1, [2, 1, 3], [900, 4100, 37], 300, seed=21))
    save_slot_case('slots_c4', *slot_case(4, [1, 2], [4200, 1500], 160, seed=22))


def grouped_golden(ref):
    """grouped_c128.npz / grouped_c4.npz: `tiled_quantized_reference(..., query_group=2 / 4)` on chunked-prefill
    shapes (several query tokens per request), reference.py:229-234,243-249,300-301."""
    for name, ratio, queries, lengths, seed in (('grouped_c128', 128, [5, 2, 1], [16500, 40000, 300], 31),
                                                ('grouped_c4', 4, [4, 3], [700, 2051], 32),
                                                # contexts within the reference's bound on grouped C4 plans (attention.py:89-98)
                                                ('grouped_c4_short', 4, [5, 2, 3, 1], [700, 1024, 131, 9], 33)):
        def duplicate(indices, g):
            indices[:, :, 40:60] = indices[:, :, 0:20]             # duplicates: multiplicity 2
            if name == 'grouped_c4_short':
                indices[:, :, 100:110] = indices[:, :, 0:10]       # and 3
        case, oq, cq = windowed_case(ref, ratio=ratio, queries=queries, lengths=lengths, seed=seed,
                                     edit_indices=duplicate if ratio == 4 else None)
        arrays = dict(q=bits(case.q), ori=case.ori.numpy(), ori_table=case.ori_block_table.numpy(), cmp=case.cmp.numpy(),
                      cmp_table=case.cmp_block_table.numpy(), cu_q=case.cu_q.numpy(), seq_lens=case.seq_lens.numpy(),
                      sink=case.sink.numpy(), ori_scale=oq.scale.numpy(), cmp_scale=cq.scale.numpy(),
                      ratio=np.int32(case.ratio), softmax_scale=np.float64(case.softmax_scale))
        if case.cmp_indices is not None:
            arrays['cmp_indices'] = case.cmp_indices.numpy()
        for group in (1, 2, 4):
            out, lse = ref.tiled_quantized_reference(case, oq, cq, tile_size=128, splits=1, query_group=group, return_lse=True)
            arrays[f'out_g{group}'] = bits(out)
            arrays[f'lse_g{group}'] = lse.numpy()
        arrays['out_s1'], arrays['lse_s1'] = arrays['out_g1'], arrays['lse_g1']
        np.savez_compressed(HERE / f'{name}.npz', **arrays)
        print(name, {k: v.shape for k, v in arrays.items() if hasattr(v, 'shape') and v.ndim}, flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument('--reference', type=Path, required=True, help='checkout of the reference project')
    parser.add_argument('--only-layout', action='store_true', help='regenerate cache_layout.json alone (needs vllm)')
    parser.add_argument('--only-slots', action='store_true', help='regenerate the explicit-slot cases alone')
    parser.add_argument('--only-grouped', action='store_true', help='regenerate the query-group cases alone')
    args = parser.parse_args()
    if args.only_layout:
        layout_golden(args.reference)
        return
    sys.path.insert(0, str(args.reference))
    from npu_sparse_attn_sharedkv_int8 import reference as ref
    if args.only_slots:
        slots_golden(ref)
        return
    if args.only_grouped:
        grouped_golden(ref)
        return
    from tests.support.serving_shapes import ActivationCorpus, Geometry

    # ---- writer: known answers and a random block (reference tests/unit/test_reference.py:22-27)
    g = torch.Generator().manual_seed(3)
    sigma = torch.exp(torch.randn(512, generator=g) * 0.5)
    rows = (torch.randn(96, 512, generator=g) * sigma).bfloat16()
    rows[0, :8] = torch.tensor([-200.0, -127.0, -1.5, -0.5, 0.5, 1.5, 127.0, 200.0]).bfloat16()
    quant = ref.CacheQuantization((rows.float().abs().amax(0) * 1.1 / 127).clamp_min(1e-8))
    unit = ref.CacheQuantization(torch.ones(512))
    kat = torch.zeros(1, 512)
    kat[0, :8] = torch.tensor([-200.0, -127.0, -1.5, -0.5, 0.5, 1.5, 127.0, 200.0])
    halves = (torch.arange(-300, 300).float() / 2).bfloat16().reshape(1, -1)      # every half-integer tie
    halves = torch.nn.functional.pad(halves, (0, 1024 - halves.shape[1])).reshape(2, 512)
    np.savez_compressed(HERE / 'writer.npz', rows=bits(rows), scale=quant.scale.numpy(),
                        inverse_scale=quant.inverse_scale.numpy(), codes=quant.quantize(rows).numpy(),
                        kat_rows=kat.numpy(), kat_codes=unit.quantize(kat).numpy(),
                        tie_rows=bits(halves), tie_codes=unit.quantize(halves).numpy())

    # ---- joint-softmax known answer (tests/unit/test_reference.py:50-56)
    q = torch.zeros(2, 512)
    caches = [torch.full((1, 512), v, dtype=torch.int8) for v in (10, 20)]
    out, lse = ref.joint_quantized_row(q, caches, [unit, unit], torch.zeros(2), 1.0)
    g = torch.Generator().manual_seed(5)
    jq = torch.randn(8, 512, generator=g).bfloat16()
    jc = [torch.randint(-127, 128, (n, 512), generator=g, dtype=torch.int8) for n in (100, 77)]
    jout, jlse = ref.joint_quantized_row(jq, jc, [quant, quant], torch.linspace(-2, 2, 8), 512 ** -0.5)
    np.savez_compressed(HERE / 'joint.npz', kat_out=bits(out), kat_lse=lse.numpy(), q=bits(jq), c0=jc[0].numpy(),
                        c1=jc[1].numpy(), scale=quant.scale.numpy(), out=bits(jout), lse=jlse.numpy())

    # ---- the reference's own unit-test geometry (tests/unit/test_reference.py:59-71)
    for ratio in (4, 128):
        case = ref.make_case(query_lengths=(2, 1), seq_lens=(129, 257), ratio=ratio, seed=23)
        oq, cq = ref.CacheQuantization.calibrate([case.ori]), ref.CacheQuantization.calibrate([case.cmp])
        save_case(f'unit_c{ratio}', replace(case, ori=oq.quantize(case.ori), cmp=cq.quantize(case.cmp)), oq, cq, ref)

    # ---- benchmark configuration 0: C4, B=2, T=1, contexts 4096 / 8192, top-k 1024, seed 0
    case, oq, cq = windowed_case(ref, ratio=4, queries=[1, 1], lengths=[4096, 8192], seed=0)
    save_case('config0_c4', case, oq, cq, ref)

    # ---- C4 selections with holes, out-of-range entries and duplicates (count >= top-k: slots keep their place)
    def damage(indices, g):
        indices[:, :, ::7] = -1
        indices[:, :, 5::11] = 2 ** 30
        indices[:, :, 3::13] = indices[:, :, 2::13][:, :, :indices[:, :, 3::13].shape[-1]]
        indices[1, :, 128:256] = -1                 # one tile with no key at all
    case, oq, cq = windowed_case(ref, ratio=4, queries=[2, 1], lengths=[4300, 4100], seed=11, edit_indices=damage)
    save_case('holes_c4', case, oq, cq, ref)

    # ---- short contexts: fewer compressed rows than top-k slots (valid selections are packed), ragged queries,
    #      a first token with no compressed row, duplicates among the packed entries
    def shuffle_short(indices, g):
        indices[0, 0, :] = indices[0, 0, torch.randperm(1024, generator=g)]
        indices[2, 0, 100:140] = indices[2, 0, 0:40]
    case, oq, cq = windowed_case(ref, ratio=4, queries=[1, 3, 1, 2], lengths=[700, 2051, 2, 131], seed=12,
                                 edit_indices=shuffle_short)
    save_case('short_c4', case, oq, cq, ref)

    # ---- C128: contexts below one compressed row, one tile, several tiles; two query tokens in one request
    case, oq, cq = windowed_case(ref, ratio=128, queries=[1, 2, 1, 1], lengths=[100, 16500, 40000, 129], seed=13)
    save_case('mixed_c128', case, oq, cq, ref)

    # ---- real activation rows with the frozen serving scales
    corpus = ActivationCorpus()
    for ratio, queries, lengths in ((4, (1, 2), (131, 1030)), (128, (2, 1), (4100, 9000))):
        source, oq, cq, _ = corpus.make(Geometry(f'real_c{ratio}', ratio, queries, lengths), layer_index=0)
        # keep only the table columns these lengths can touch
        case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp),
                       ori_block_table=source.ori_block_table[:, :math.ceil(max(lengths) / 32)].contiguous(),
                       cmp_block_table=source.cmp_block_table[:, :max(1, math.ceil(max(lengths) / (ratio * 32)))].contiguous())
        save_case(f'real_c{ratio}', case, oq, cq, ref)

    slots_golden(ref)
    grouped_golden(ref)

    layout_golden(args.reference)


if __name__ == '__main__':
    main()
