"""The decode entry point for callers that cannot allocate (``itk_decode_attention_noalloc``).

Some users of this library run where device allocation is not allowed at call time: a server that reserved
all of its memory at start-up, a plugin inside another runtime that owns the allocator, a latency-critical
loop that cannot take cudaMalloc's synchronisation, or work that is being recorded for replay.  For them the
library offers one decode-attention call whose split-K scratch is a fixed array built into the library, so
the call itself allocates nothing.  This test drives that call through the C ABI, twice in a row (the array
is shared and keeps the previous call's contents), and checks it against the ordinary backend call on the
same cache contents and against the CPU oracle's attention over the same (f16-rounded) rows, to the tolerance
the other attention tests use.  It also checks that a request beyond the array's stated capacity is refused
with a message instead of being run.

The file sorts last on purpose: if it fails, a run that stops at the first failure has already run
everything else.
"""
import ctypes as C

import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, KvDtype, _lib

from kvparity import TOL_F16_KV, attention_error
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def call_noalloc(lib, k_dev, v_dev, ring, hkv, hq, d, slots, lens, q_dev, out_dev, splits, stream):
    n = len(slots)
    sl = (C.c_uint32 * max(n, 1))(*slots)
    ln = (C.c_uint32 * max(n, 1))(*lens)
    err = C.create_string_buffer(256)
    rc = lib.itk_decode_attention_noalloc(C.c_void_p(k_dev.data_ptr()), C.c_void_p(v_dev.data_ptr()), ring, hkv, hq, d,
                                          n, sl, ln, C.c_void_p(q_dev.data_ptr()), C.c_void_p(out_dev.data_ptr()),
                                          splits, C.c_void_p(stream), err, len(err))
    return rc, err.value.decode()


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (8, 2, 64)])
def test_noalloc_decode_matches_the_backend_call_twice_in_a_row(hq, hkv, d):
    import torch

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    lens = [700, 64, 1531]
    n_slots, ring = len(lens), 1600
    rng = np.random.default_rng(hq * 1000 + d)

    # The ordinary path: a backend that owns its cache (and allocates it).
    gpu = CudaCompute(1, hq, hkv, d, n_slots=n_slots, max_context=ring, chunk_cap=1, kv_dtype=KvDtype.F16)
    # The caller-owned cache for the new call: same rows, this library's layout [slot][kv_head][row][D], f16.
    k_dev = torch.zeros((n_slots, hkv, ring, d), dtype=torch.float16, device=dev)
    v_dev = torch.zeros_like(k_dev)
    refs = []
    for slot, n in enumerate(lens):
        k = rng.standard_normal((n, hkv, d)).astype(np.float32)
        v = rng.standard_normal((n, hkv, d)).astype(np.float32)
        gpu.append_rows(0, k, v, 0, slot=slot)
        ref = orc.KvCache([orc.GLOBAL], hkv, d)
        ref.append_rows(0, orc.round_through_f16(k.reshape(n, -1)), orc.round_through_f16(v.reshape(n, -1)), 0)
        refs.append(ref)
        k_dev[slot, :, :n] = torch.from_numpy(k).to(dev).permute(1, 0, 2).to(torch.float16)
        v_dev[slot, :, :n] = torch.from_numpy(v).to(dev).permute(1, 0, 2).to(torch.float16)
    stream = torch.cuda.current_stream().cuda_stream
    out_dev = torch.empty((n_slots, hq * d), dtype=torch.float32, device=dev)

    # Two calls in a row with different queries and split counts: the second starts from whatever the first
    # left in the shared array.
    for call, splits in enumerate((0, 5)):
        q = rng.standard_normal((n_slots, hq * d)).astype(np.float32)
        want = np.stack([gpu.gqa_attention(0, q[s], [lens[s] - 1], slot=s) for s in range(n_slots)])
        q_dev = torch.from_numpy(q).to(dev)
        out_dev.fill_(float("nan"))
        rc, msg = call_noalloc(lib, k_dev, v_dev, ring, hkv, hq, d, list(range(n_slots)), lens, q_dev, out_dev, splits,
                               stream)
        assert rc == _lib.OK, msg
        torch.cuda.synchronize()
        got = out_dev.cpu().numpy()
        assert np.all(np.isfinite(got)), f"call {call}: non-finite output"
        err = attention_error(got, want, hq, d)
        assert err <= TOL_F16_KV, f"call {call}: differs from the backend call by {err:.3e} of the output norm"
        oracle_out = np.stack([orc.gqa_attention(q[s], 1, hq, [lens[s] - 1], refs[s].view(0)) for s in range(n_slots)])
        err = attention_error(got, oracle_out, hq, d)
        assert err <= TOL_F16_KV, f"call {call}: differs from the CPU oracle by {err:.3e} of the output norm"

    # Beyond the built-in array: refused by name, nothing launched.
    rc, msg = call_noalloc(lib, k_dev, v_dev, ring, hkv, hq, d, list(range(n_slots)), lens, q_dev, out_dev, 4096, stream)
    assert rc == _lib.ERR_CAPACITY and "splits exceed" in msg
    # cells x max(splits, 2) is the bound: with one split, 64 sequences x 18 KV heads = 1152 cells need 2304 slots
    rc, msg = call_noalloc(lib, k_dev, v_dev, ring, 18, 18, d, [0] * 64, [1] * 64, q_dev, out_dev, 1, stream)
    assert rc == _lib.ERR_CAPACITY and "exceeds the built-in scratch" in msg
    # a misaligned query pointer is refused, not dereferenced
    err_buf = C.create_string_buffer(256)
    sl, ln = (C.c_uint32 * 1)(0), (C.c_uint32 * 1)(10)
    rc = lib.itk_decode_attention_noalloc(C.c_void_p(k_dev.data_ptr()), C.c_void_p(v_dev.data_ptr()), ring, hkv, hq, d, 1,
                                          sl, ln, C.c_void_p(q_dev.data_ptr() + 4), C.c_void_p(out_dev.data_ptr()), 1,
                                          C.c_void_p(stream), err_buf, len(err_buf))
    assert rc == _lib.ERR_INVALID_ARGUMENT and b"16-byte aligned" in err_buf.value
    rc, msg = call_noalloc(lib, k_dev, v_dev, ring, hkv, hq, d, [0] * 65, [1] * 65, q_dev, out_dev, 1, stream)
    assert rc == _lib.ERR_CAPACITY and "maximum of 64" in msg
    rc, msg = call_noalloc(lib, k_dev, v_dev, ring, hkv, hq, 96, [0], [10], q_dev, out_dev, 1, stream)
    assert rc == _lib.ERR_CAPACITY and "head_dim" in msg
    torch.cuda.synchronize()
