"""GPU: tq_decode_attn_static, the entry point for hosts that may not allocate while running
(their scratch comes from an array built into the library), must give the same answer as
tq_decode_attn with a caller workspace.  Collected last so that a stop-at-first-failure run
has already exercised everything else."""

from __future__ import annotations

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _decode_static(store, q, splits):
    from tq_local_b200.runtime import ffi
    from tq_local_b200.runtime.codec import tq_dtype

    b, hq = q.shape[0], q.shape[1]
    qc = q.reshape(b, hq, 128).contiguous()
    out = torch.empty(b, hq, 1, 128, dtype=q.dtype, device=q.device)
    with torch.cuda.device(q.device):
        rc = ffi.lib().tq_decode_attn_static(store.codec.handle, qc.data_ptr(), tq_dtype(q.dtype), hq,
                                             C.byref(store._desc), store.length, splits, out.data_ptr(),
                                             C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
    return rc, out


@pytest.mark.parametrize("dtype,hq", [(torch.bfloat16, 8), (torch.float32, 8), (torch.float16, 14)])
def test_static_scratch_entry_matches_workspace_entry(dtype, hq):
    from tq_local_b200.runtime import ffi
    from tq_local_b200.runtime.codec import Codec
    from tq_local_b200.runtime.packed_store import PackedStore

    dev = torch.device("cuda", torch.cuda.current_device())
    codec = Codec.get(dev, 4, True)
    gen = torch.Generator(device=dev).manual_seed(5)
    n = 1500
    k = torch.randn(2, 2, n, 128, device=dev, generator=gen).to(dtype)
    v = torch.randn(2, 2, n, 128, device=dev, generator=gen).to(dtype)
    store = PackedStore(codec, 2, 2, capacity=n)
    store.pack(k, v)
    assert ffi.lib().tq_static_scratch_bytes() == 8 << 20
    # two calls in a row with different queries: the shared array carries no state between them
    for seed in (1, 2):
        q = torch.randn(2, hq, 1, 128, device=dev, generator=torch.Generator(device=dev).manual_seed(seed)).to(dtype)
        want = store.decode_attn(q, splits=3)
        rc, got = _decode_static(store, q, 3)
        torch.cuda.synchronize()
        assert rc == 0
        torch.testing.assert_close(got.float(), want.float(), rtol=0, atol=1e-6 * float(want.float().abs().max()))
    assert codec.device_status() == 0


def test_static_scratch_entry_rejects_oversized_shapes():
    from tq_local_b200.runtime import ffi
    from tq_local_b200.runtime.codec import Codec
    from tq_local_b200.runtime.packed_store import PackedStore

    dev = torch.device("cuda", torch.cuda.current_device())
    codec = Codec.get(dev, 4, True)
    store = PackedStore(codec, 8, 8, capacity=64)
    x = torch.zeros(8, 8, 64, 128, device=dev, dtype=torch.bfloat16)
    store.pack(x, x)
    q = torch.zeros(8, 32, 1, 128, device=dev, dtype=torch.bfloat16)
    assert ffi.lib().tq_decode_workspace_bytes(8, 32, 256) > 8 << 20
    rc, _ = _decode_static(store, q, 256)
    assert rc == -4  # TQ_ERR_WORKSPACE
    assert b"8 MiB" in ffi.lib().tq_last_cuda_error()
    rc, _ = _decode_static(store, q, 4)
    torch.cuda.synchronize()
    assert rc == 0
