"""The SGLang backend class end to end on the GPU, over stand-ins for SGLang: the chunk is written
through to the pool, both requests of a forward run through the native batched entry, and the result is
byte-identical to calling the operator per request, as the reference's backend loop does
(engines/sglang/integration/fp8_prefill/backend.py:226-291)."""
import numpy as np
import pytest
import torch

import akl_oracle as O
import helpers as H
import sglang_stubs as S

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qk", ["fp8", "int8"])
def test_forward_extend_equals_per_request_operator_calls(pkg, cuda, monkeypatch, qk):
    from attn_kernel_lab_b200 import backend

    monkeypatch.setenv("SGLANG_FP8_PREFILL_MIN_TOKENS", "64")
    monkeypatch.setenv("SGLANG_FP8_PREFILL_QK", qk)
    for key in ("DISABLE", "BF16_HEADS", "MIN_EXTEND", "K_CENTER", "HADAMARD"):
        monkeypatch.delenv("SGLANG_FP8_PREFILL_" + key, raising=False)
    cls = backend.make_backend_class(S.BaseBackend, S.ForwardMode.EXTEND)
    g = torch.Generator().manual_seed(77)
    prefix, extend, slots, Hq, Hkv = (700, 130), (200, 333), 8192, 24, 4
    pool = S.KVPool(slots, Hkv, 3, cuda)
    perm = torch.randperm(slots, generator=g)
    table = torch.zeros(3, 1024, dtype=torch.int32)
    at = 0
    for r, n in enumerate(p + e for p, e in zip(prefix, extend)):
        table[r + 1, :n] = perm[at:at + n].to(torch.int32)
        at += n
    # cached prefixes are already in the pool (layer 2); the chunk's K/V arrive with the call
    for r, p in enumerate(prefix):
        rows = table[r + 1, :p].long().to(cuda)
        pool.k[2][rows] = torch.randn(p, Hkv, 256, generator=g).to(torch.bfloat16).to(cuda)
        pool.v[2][rows] = torch.randn(p, Hkv, 256, generator=g).to(torch.bfloat16).to(cuda)
    be = cls(S.model_runner(pool, table.to(cuda)))
    new_rows = torch.cat([table[r + 1, p:p + e] for r, (p, e) in enumerate(zip(prefix, extend))]).to(cuda)
    fb = S.ForwardBatch(S.ForwardMode.EXTEND, list(prefix), list(extend),
                        torch.arange(1, 3, device=cuda), new_rows)
    layer = S.Layer(layer_id=2)
    tokens = sum(extend)
    q = torch.randn(tokens, Hq * 256, generator=g).to(torch.bfloat16).to(cuda)
    k = torch.randn(tokens, Hkv * 256, generator=g).to(torch.bfloat16).to(cuda)
    v = torch.randn(tokens, Hkv * 256, generator=g).to(torch.bfloat16).to(cuda)

    be.init_forward_metadata(fb)
    out = be.forward_extend(q, k, v, layer, fb)
    torch.cuda.synchronize()
    assert be.fallback_calls == [] and pool.writes == [(2, tokens)]
    assert out.shape == q.shape and out.dtype == torch.bfloat16

    q3, row0 = q.view(tokens, Hq, 256), 0
    for r, (p, e) in enumerate(zip(prefix, extend)):
        idx = table[r + 1, :p + e].long().to(cuda)
        want, lse = pkg.prefill_extend(q3[row0:row0 + e], pool.k[2], pool.v[2], idx, p,
                                       sm_scale=layer.scaling, return_lse=True, qk_i8=qk == "int8")
        torch.cuda.synchronize()
        got = out.view(tokens, Hq, 256)[row0:row0 + e]
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"request {r}"
        if r == 1:      # and the operator itself against the float64 oracle, once
            ref = O.reference(q3[row0:row0 + e].float().cpu().numpy(), pool.k[2][idx].float().cpu().numpy(),
                              pool.v[2][idx].float().cpu().numpy(), p, sm_scale=layer.scaling,
                              qk_i8=qk == "int8")
            rel = H.row_rel(got.float().cpu().numpy(), ref)
            assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() > 0.97
        row0 += e
