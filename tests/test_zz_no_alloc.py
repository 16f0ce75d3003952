"""The decode-attention entry point that allocates nothing (csrc/kernels/attention_decode_static.h).

It serves callers that cannot allocate device memory (a process whose GPU memory is wholly owned
by its own arena, or code that must not trigger cudaMalloc's device-wide synchronisation mid-step):
the split partial results go to an array inside the library image instead of a caller's buffer.
The test calls it through its exported C symbol, twice in a row with different shapes so that the
second call finds the first one's leftovers in the shared array, and compares each result with
the ordinary entry point's (which gets a scratch buffer from the caller).

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from rust_llm_inference_server_b200.ops import build
    lib = ctypes.CDLL(build.build_kernels())
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    static = lib.rlis_attention_decode_static
    static.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P]
    static.restype = I
    plain = lib.rlis_attention_decode
    plain.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P]
    plain.restype = I
    cap = lib.rlis_attention_decode_static_capacity
    cap.restype = ctypes.c_longlong
    return static, plain, cap


def _case(nh, nkv, d, ps, lens, seed):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    n_pages = sum((n + ps - 1) // ps for n in lens) + 2
    kc = torch.randn(n_pages, nkv, ps, d, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(n_pages, nkv, ps, d, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(B, nh * d, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max((n + ps - 1) // ps for n in lens)
    tables = torch.full((B, width), -1, dtype=torch.int32)
    for b, n in enumerate(lens):
        for i in range((n + ps - 1) // ps):
            tables[b, i] = perm.pop()
    rows = torch.arange(B, dtype=torch.int32).cuda()
    return q, kc, vc, tables.cuda(), rows, torch.tensor(lens, dtype=torch.int32).cuda()


def test_static_entry_point_equals_the_ordinary_one_on_two_calls_in_a_row():
    static, plain, cap = _symbols()
    assert cap() == 2 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    # the second call is smaller than the first (fewer requests, fewer splits): whatever the first
    # call left in the shared array lies beside and under what the second one writes
    calls = [((32, 8, 64, 16), [900, 2049, 33, 1, 700, 1500], 7, 1),
             ((6, 3, 48, 8), [300, 77], 3, 2),
             ((32, 8, 64, 16), [4096], 1, 3)]
    for (nh, nkv, d, ps), lens, splits, seed in calls:
        q, kc, vc, tables, rows, ctx = _case(nh, nkv, d, ps, lens, seed)
        B = len(lens)
        scale = 1.0 / math.sqrt(d)
        want = torch.zeros(B, nh * d, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(B * nh * splits * (d + 2), dtype=torch.float32, device="cuda")
        rc = plain(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), want.data_ptr(), scratch.data_ptr(),
                   rows.data_ptr(), rows.data_ptr(), ctx.data_ptr(), tables.data_ptr(), tables.shape[1],
                   B, nh, nkv, d, ps, scale, 0, splits, 1, stream)
        assert rc == 0
        got = torch.zeros_like(want)
        rc = static(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), got.data_ptr(), rows.data_ptr(),
                    rows.data_ptr(), ctx.data_ptr(), tables.data_ptr(), tables.shape[1], B, nh, nkv, d, ps,
                    scale, 0, splits, 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # the same kernels on the same inputs: within the tolerance of the kernel tests (and in
        # fact bit for bit, since only the scratch's address differs)
        assert (got.float() - want.float()).abs().max() <= 2e-2
        assert torch.equal(got, want)


def test_static_entry_point_refuses_more_than_its_array_holds():
    static, _, cap = _symbols()
    nh, nkv, d, ps, splits = 32, 8, 64, 16, 64
    B = int(cap()) // (nh * splits * (d + 2)) + 1
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    # nothing is launched and nothing is dereferenced: the size check comes first
    rc = static(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                z.data_ptr(), z.data_ptr(), 1, B, nh, nkv, d, ps, 0.125, 0, splits, 1,
                torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    torch.cuda.synchronize()
