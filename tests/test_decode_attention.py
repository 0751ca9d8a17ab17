"""Split-KV decode attention kernel against NumPy on a synthetic cache (bf16 and fp32), with
ragged context lengths that end inside a 16-key block, inside a CTA's key range and across
several splits."""
import ctypes as C

import numpy as np
import pytest

import luminal_oracle as O

pytestmark = pytest.mark.gpu


def synth_cache(cfg, batch, max_ctx, n_pos, layer, seed):
    KV, D = cfg["n_kv_heads"], cfg["hidden"] // cfg["n_heads"]
    k = O.synth_normal(seed, 0x100000 + 2 * layer, (batch, KV, max_ctx, D), 1.0)[:, :, :n_pos]
    v = O.synth_normal(seed, 0x100000 + 2 * layer + 1, (batch, KV, max_ctx, D), 1.0)[:, :, :n_pos]
    return k, v


def ref_attention(q, k, v, n_heads, n_kv):
    """q [B,H,D] in the reference's head order; kv head of q head h is h mod KV (src/NN.jl:305-317)."""
    B, H, D = q.shape
    out = np.empty_like(q)
    for h in range(H):
        kk, vv = k[:, h % n_kv], v[:, h % n_kv]                  # [B,T,D]
        s = np.einsum("bd,btd->bt", q[:, h].astype(np.float64), kk.astype(np.float64)) / np.sqrt(D)
        s -= s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=1, keepdims=True)
        out[:, h] = np.einsum("bt,btd->bd", p, vv.astype(np.float64))
    return out


@pytest.mark.parametrize("dtype,tol", [("bf16", 2e-2), ("f32", 1e-5)])
@pytest.mark.parametrize("name,batch,max_ctx,Ts", [
    ("tiny_gqa128", 3, 700, [1, 15, 16, 17, 333, 700]),
    ("tiny_gqa96", 2, 200, [5, 64, 129, 200]),
    ("small_llama", 2, 96, [33, 96]),
])
def test_decode_attention_matches_numpy(lib_built, device, dtype, tol, name, batch, max_ctx, Ts):
    import torch
    L = lib_built
    cfg = O.CONFIGS[name]
    H, KV, D = cfg["n_heads"], cfg["n_kv_heads"], cfg["hidden"] // cfg["n_heads"]
    G = H // KV
    model = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=H, n_kv_heads=KV,
                    intermediate=cfg["intermediate"], vocab=cfg["vocab"], dtype=dtype)
    sess = L.Session(model, batch, max_ctx)
    sess.fill_kv_random(max_ctx, seed=99)
    layer = cfg["n_layers"] - 1
    k, v = synth_cache(cfg, batch, max_ctx, max_ctx, layer, 99)
    if dtype == "bf16":
        k, v = O.bf16_round(k), O.bf16_round(v)
    q = O.synth_normal(5, 77, (batch, H, D), 1.0)
    if dtype == "bf16":
        q = O.bf16_round(q)
    # library order of the local q heads: (kv head, group) -> reference head kv + KV*g
    order = [kvh + KV * g for kvh in range(KV) for g in range(G)]
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    q_dev = torch.tensor(q[:, order, :], device="cuda").to(tdt).contiguous()
    out_dev = torch.empty_like(q_dev)
    torch.cuda.synchronize()
    for T in Ts:
        sess.decode_attention(layer, q_dev.data_ptr(), out_dev.data_ptr(), T)
        device.sync()
        got = np.empty_like(q)
        got[:, order, :] = out_dev.float().cpu().numpy()
        ref = ref_attention(q, k[:, :, :T], v[:, :, :T], H, KV)
        err = np.abs(got - ref).max() / (np.abs(ref).max() + 1e-30)
        assert err <= tol, f"T={T}: {err}"
    sess.close(); model.close()
