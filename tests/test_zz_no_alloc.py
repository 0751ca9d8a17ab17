"""The allocation-free decode-attention entry point against the regular one and against NumPy.

Some users of this library cannot let it call cudaMalloc -- their own runtime already owns the
whole device in a memory pool, or they sit in a loop where an allocation's implicit
synchronisation is not acceptable.  lmb200_decode_attention_noalloc keeps the kernel's split-KV
partials in an array compiled into the library instead.  This test calls it twice in a row
through the C ABI on the same cache and checks both results against
lmb200_decode_attention_splitkv (which uses scratch the session allocated) and against a float64
NumPy attention over the same regenerated cache, within the tolerance of the decode-attention
tests.  It lives in a file that pytest collects last, so a run that stops at the first failure
has already run everything else."""
import numpy as np
import pytest

import luminal_oracle as O

from test_decode_attention import ref_attention, synth_cache

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [("bf16", 2e-2), ("f32", 1e-5)])
def test_noalloc_attention_matches_session_attention(lib_built, device, dtype, tol):
    import torch
    L = lib_built
    cfg = O.CONFIGS["tiny_gqa128"]
    H, KV, D = cfg["n_heads"], cfg["n_kv_heads"], cfg["hidden"] // cfg["n_heads"]
    G = H // KV
    batch, max_ctx = 3, 600
    model = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=H, n_kv_heads=KV,
                    intermediate=cfg["intermediate"], vocab=cfg["vocab"], dtype=dtype)
    sess = L.Session(model, batch, max_ctx)
    sess.fill_kv_random(max_ctx, seed=5)
    layer = 1
    kv_ptr, bstride, hstride = sess.kv_layer(layer)
    k, v = synth_cache(cfg, batch, max_ctx, max_ctx, layer, 5)
    if dtype == "bf16":
        k, v = O.bf16_round(k), O.bf16_round(v)
    # library order of the q heads: (kv head, group member) -> reference head kv + KV*g
    order = [kvh + KV * g for kvh in range(KV) for g in range(G)]
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    for call, T in enumerate((600, 333)):          # two calls in a row share the built-in array
        q_ref = O.synth_normal(call, 77, (batch, H, D), 1.0)
        if dtype == "bf16":
            q_ref = O.bf16_round(q_ref)
        q = torch.tensor(q_ref[:, order, :], device="cuda").to(tdt).contiguous()
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        sess.decode_attention(layer, q.data_ptr(), want.data_ptr(), T)
        L.decode_attention_noalloc(device, dtype, q.data_ptr(), got.data_ptr(), kv_ptr, bstride, hstride,
                                   batch, KV, G, D, T)
        device.sync()
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.isfinite(g).all()
        assert np.abs(g - w).max() / (np.abs(w).max() + 1e-30) <= tol, f"call {call}, T={T}: differs from the session entry"
        ref = ref_attention(q_ref, k[:, :, :T], v[:, :, :T], H, KV)
        g_ref_order = np.empty_like(q_ref)
        g_ref_order[:, order, :] = g
        err = np.abs(g_ref_order - ref).max() / (np.abs(ref).max() + 1e-30)
        assert err <= tol, f"call {call}, T={T}: differs from NumPy by {err}"
    # a context longer than the strides can hold is refused before anything is launched
    with pytest.raises(L.LuminalB200Error, match="kv head stride"):
        L.decode_attention_noalloc(device, dtype, q.data_ptr(), got.data_ptr(), kv_ptr, bstride, hstride,
                                   batch, KV, G, D, max_ctx + 64 + 1)
    with pytest.raises(L.LuminalB200Error, match="batch stride"):
        L.decode_attention_noalloc(device, dtype, q.data_ptr(), got.data_ptr(), kv_ptr, hstride, hstride,
                                   batch, KV, G, D, 100)
    # a shape whose partials do not fit the built-in array is refused, not truncated (strides that
    # would be valid for it, so that the scratch check is the one that answers; nothing is launched)
    big_T = 600 * 10**6 // 64 * 64
    big_h = (big_T // 16) * 32 * D
    with pytest.raises(L.LuminalB200Error, match="scratch floats"):
        L.decode_attention_noalloc(device, dtype, q.data_ptr(), got.data_ptr(), kv_ptr, big_h * KV, big_h,
                                   batch, KV, G, D, big_T)
    sess.close(); model.close()
