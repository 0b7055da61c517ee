"""The allocation-free split decode against the ordinary entry point (collected last on purpose).

`mla_sparse_decode_noalloc_launcher` serves callers that cannot pass scratch memory: processes whose
allocator is closed on the request path, or operator interfaces with inputs and outputs only. Its
partial results go to a fixed array inside the library, so the test checks, through the C ABI, that
two consecutive calls (different inputs, so stale partials would show) give what the ordinary entry
point gives with caller-provided scratch, at the tolerance the MLA tests use (atol 2e-2), and that an
oversized request is refused before anything is launched.
"""
import pytest
import torch

from conftest import load_oracle

ATOL = 2e-2


@pytest.mark.gpu
def test_noalloc_entry_matches_ordinary_entry_twice(cuda_device):
    from cuda_agent_b200 import capi
    dev = cuda_device
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    B, Hh, S, topk, nsplit = 2, 128, 3000, 1024, 4
    assert B * nsplit * Hh * 2056 <= capi.MLA_STATIC_SCRATCH_BYTES
    scratch = torch.empty(capi.mla_scratch_bytes(B, Hh, nsplit), dtype=torch.uint8, device=dev)
    for call in range(2):
        gen = torch.Generator().manual_seed(50 + call)
        q, kv, seq_len, idx = [t.to(dev) for t in m.make_inputs(B, Hh, S, topk, 900, gen)]
        if call == 1:
            idx[0, 0, ::3] = -1                      # fewer valid rows than in the first call
        expect = torch.full((B, 1, Hh, 512), float("nan"), dtype=torch.bfloat16, device=dev)
        got = torch.full_like(expect, float("nan"))
        st = torch.ones(2, dtype=torch.int32, device=dev)
        capi.mla_sparse_decode(expect, q, kv, seq_len, idx, 192 ** -0.5, nsplit, scratch, st[0:1])
        capi.mla_sparse_decode_noalloc(got, q, kv, seq_len, idx, 192 ** -0.5, nsplit, st[1:2])
        torch.cuda.synchronize()
        assert st.cpu().tolist() == [0, 0]
        assert torch.isfinite(got.float()).all()
        assert float((got.float() - expect.float()).abs().max()) <= ATOL
        ref = m.Model(B, Hh, S, topk)(q.cpu(), kv.cpu(), seq_len.cpu(), idx.cpu())
        assert float((got.cpu().float() - ref.float()).abs().max()) <= ATOL


@pytest.mark.gpu
def test_noalloc_entry_rejects_what_does_not_fit(cuda_device):
    from cuda_agent_b200 import capi
    dev = cuda_device
    B, Hh, nsplit = 64, 128, 2                        # 64 * 2 * 128 * 2056 B = 33.7 MB > 16 MiB
    assert B * nsplit * Hh * 2056 > capi.MLA_STATIC_SCRATCH_BYTES
    tiny = torch.zeros(16, dtype=torch.bfloat16, device=dev)      # never dereferenced: refused on the host
    ints = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = capi.lib().mla_sparse_decode_noalloc_launcher(tiny.data_ptr(), tiny.data_ptr(), tiny.data_ptr(),
                                                       ints.data_ptr(), ints.data_ptr(), B, Hh, 1024, 2048, 0.07,
                                                       nsplit, None, 0, None)
    assert rc == 4 and "exceeds" in capi.status_string(rc)
    with pytest.raises(capi.CabError):
        capi.mla_sparse_decode_noalloc(torch.empty(B, 1, Hh, 512, dtype=torch.bfloat16, device=dev),
                                       torch.empty(B, 1, Hh, 576, dtype=torch.bfloat16, device=dev),
                                       torch.empty(B, 8, 576, dtype=torch.bfloat16, device=dev),
                                       torch.zeros(B, dtype=torch.int32, device=dev),
                                       torch.zeros(B, 1, 64, dtype=torch.int32, device=dev), 0.07, nsplit)
    torch.cuda.synchronize()
