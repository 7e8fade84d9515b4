"""The no-allocation single-token attention entry point, called through its exported C symbol.

``lse_attn_decode_noalloc`` serves callers that may not allocate device memory (a host program
whose own pool already holds all of it, a serving loop that must never hit cudaMalloc's
device-wide synchronisation): the partial results of the context partitions go to a buffer inside
the library's device image instead of a caller-allocated one. This test loads the attention
library for head size 64 with ctypes, runs the new entry point and the existing one
(``lse_attn_decode``, scratch allocated here with torch) on the same inputs, twice in a row with
different inputs, and compares the outputs. The file sorts last so that a run that stops at the
first failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

D, PAGE, NQ, NK = 64, 16, 6, 2


class AttnArgs(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int), ("q", ctypes.c_void_p), ("q_row_stride", ctypes.c_longlong),
        ("out", ctypes.c_void_p), ("out_row_stride", ctypes.c_longlong),
        ("k_pages", ctypes.c_void_p), ("v_pages", ctypes.c_void_p),
        ("num_heads", ctypes.c_int), ("num_kv_heads", ctypes.c_int), ("page_tokens", ctypes.c_int),
        ("window", ctypes.c_int), ("scale", ctypes.c_float),
        ("block_tables", ctypes.c_void_p), ("table_stride", ctypes.c_int),
        ("ctx_lens", ctypes.c_void_p), ("cu_q", ctypes.c_void_p),
        ("tiles", ctypes.c_void_p), ("num_tiles", ctypes.c_int), ("force_simt", ctypes.c_int),
        ("decode_seqs", ctypes.c_void_p), ("num_decode", ctypes.c_int), ("num_splits", ctypes.c_int),
        ("scratch", ctypes.c_void_p),
        ("num_rows", ctypes.c_longlong), ("num_pages", ctypes.c_longlong), ("error_flag", ctypes.c_void_p),
        ("qkv_sums", ctypes.c_void_p), ("rope_cos", ctypes.c_void_p), ("rope_sin", ctypes.c_void_p),
    ]


@pytest.fixture(scope="module")
def lib():
    from llmserve_b200.ops import build

    so = ctypes.CDLL(build.attention_library(D))
    for name in ("lse_attn_decode", "lse_attn_decode_noalloc"):
        fn = getattr(so, name)
        fn.argtypes = [ctypes.POINTER(AttnArgs), ctypes.c_void_p]
        fn.restype = ctypes.c_int
    so.lse_attn_decode_noalloc_max_floats.restype = ctypes.c_size_t
    so.lse_attn_decode_scratch_floats.argtypes = [ctypes.c_int] * 3
    so.lse_attn_decode_scratch_floats.restype = ctypes.c_size_t
    return so


def make_case(seed, dtype, ctx_lens, splits):
    g = torch.Generator().manual_seed(seed)
    B = len(ctx_lens)
    blocks = [-(-c // PAGE) for c in ctx_lens]
    pages = sum(blocks) + 2
    tables = torch.zeros(B, max(blocks), dtype=torch.int32)
    order = iter(torch.randperm(pages, generator=g).tolist())
    for s in range(B):
        for b in range(blocks[s]):
            tables[s, b] = next(order)
    dev = "cuda"
    t = dict(
        q=torch.randn(B, NQ * D, generator=g).to(dtype).to(dev),
        k=torch.randn(pages, NK, PAGE, D, generator=g).to(dtype).to(dev),
        v=torch.randn(pages, NK, PAGE, D, generator=g).to(dtype).to(dev),
        tables=tables.to(dev), ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=dev),
        cu=torch.arange(B + 1, dtype=torch.int32, device=dev),
        seqs=torch.arange(B, dtype=torch.int32, device=dev),
    )
    t["B"], t["splits"], t["dtype"] = B, splits, dtype
    return t


def args_for(t, out, scratch):
    a = AttnArgs()
    a.dtype = 0 if t["dtype"] == torch.float32 else 1
    a.q, a.q_row_stride = t["q"].data_ptr(), NQ * D
    a.out, a.out_row_stride = out.data_ptr(), NQ * D
    a.k_pages, a.v_pages = t["k"].data_ptr(), t["v"].data_ptr()
    a.num_heads, a.num_kv_heads, a.page_tokens, a.window, a.scale = NQ, NK, PAGE, 0, D**-0.5
    a.block_tables, a.table_stride = t["tables"].data_ptr(), t["tables"].shape[1]
    a.ctx_lens, a.cu_q = t["ctx"].data_ptr(), t["cu"].data_ptr()
    a.tiles, a.num_tiles, a.force_simt = None, 0, 0
    a.decode_seqs, a.num_decode, a.num_splits = t["seqs"].data_ptr(), t["B"], t["splits"]
    a.scratch = scratch.data_ptr() if scratch is not None else None
    a.num_rows, a.num_pages, a.error_flag = t["B"], t["k"].shape[0], None
    return a


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_point_matches_the_allocating_one_twice_in_a_row(lib, dtype):
    stream = torch.cuda.current_stream().cuda_stream
    tol = 1e-6 if dtype == torch.float32 else 0.0  # same kernels, same order of operations
    for call, (seed, ctx_lens, splits) in enumerate([(1, [700, 33, 1, 250], 7), (2, [90, 513], 3)]):
        t = make_case(seed, dtype, ctx_lens, splits)
        need = lib.lse_attn_decode_scratch_floats(t["B"], NQ, splits)
        assert 0 < need <= lib.lse_attn_decode_noalloc_max_floats()
        ref = torch.zeros(t["B"], NQ * D, dtype=dtype, device="cuda")
        scratch = torch.zeros(need, dtype=torch.float32, device="cuda")  # its counters start at zero
        assert lib.lse_attn_decode(ctypes.byref(args_for(t, ref, scratch)), stream) == 0
        got = torch.full_like(ref, 7.0)
        assert lib.lse_attn_decode_noalloc(ctypes.byref(args_for(t, got, None)), stream) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert (got.float() - ref.float()).abs().max().item() <= tol, f"call {call}"
        # and both agree with a direct softmax over the gathered keys
        for s, c in enumerate(ctx_lens):
            j = torch.arange(c, device="cuda")
            pg = t["tables"][s, j // PAGE].long()
            k = t["k"][pg, :, j % PAGE].float().repeat_interleave(NQ // NK, dim=1)
            v = t["v"][pg, :, j % PAGE].float().repeat_interleave(NQ // NK, dim=1)
            sc = torch.einsum("hd,shd->hs", t["q"][s].float().view(NQ, D), k) * D**-0.5
            want = torch.einsum("hs,shd->hd", sc.softmax(-1), v).reshape(-1)
            bound = 1e-5 if dtype == torch.float32 else 0.02 * want.abs().max().item()
            assert (got[s].float() - want).abs().max().item() <= bound


def test_no_alloc_entry_point_refuses_what_does_not_fit(lib):
    t = make_case(3, torch.bfloat16, [64] * 4, 2)
    out = torch.zeros(t["B"], NQ * D, dtype=torch.bfloat16, device="cuda")
    a = args_for(t, out, None)
    a.num_decode, a.num_splits = 60000, 64  # 60000 * 6 * 64 * 66 floats: far beyond the buffer
    assert lib.lse_attn_decode_noalloc(ctypes.byref(a), torch.cuda.current_stream().cuda_stream) == 3
    torch.cuda.synchronize()
    assert torch.equal(out, torch.zeros_like(out))  # nothing ran
