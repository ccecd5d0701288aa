"""Generates the committed fixtures in this directory.

    python tests/golden/make_golden.py

Expected values come from torch's own operators on fp32-upcast inputs -- ``torch.mm`` and
``torch.nn.functional.scaled_dot_product_attention`` -- i.e. the operators the reference's GEMM
export and SDPA rewrites call (iree/turbine/kernel/boo/op_exports/gemm.py:217-230,
iree/turbine/kernel/boo/fusion/replacement.py:239-290), NOT from the oracle under test.  The
paged fixtures' expected values come from an explicit per-token Python loop over the block table.
Inputs are stored as raw 16-bit patterns so the files are bit-stable.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle  # noqa: E402  (input generators only)


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def gemm_case():
    a, b = oracle.make_gemm_inputs(96, 80, 64, torch.float16, seed=10)
    c = torch.mm(a.float(), b.float().t())
    np.savez_compressed(os.path.join(HERE, "gemm_f16_96x80x64.npz"), a=bits16(a), b=bits16(b), c=c.numpy())


def attention_cases():
    for name, causal, sq, skv, hq, hkv, dtype in [
        ("attn_f16_noncausal", False, 72, 200, 2, 2, torch.float16),
        ("attn_bf16_causal_gqa", True, 160, 160, 2, 1, torch.bfloat16),
        ("attn_f16_causal_offset", True, 40, 136, 2, 1, torch.float16),
    ]:
        q, k, v = oracle.make_attention_inputs(1, hq, hkv, sq, skv, 128, dtype, seed=11, std=0.5 if causal else 1.0)
        scale = 128 ** -0.5
        g = hq // hkv
        kf = k.float().repeat_interleave(g, dim=1)
        vf = v.float().repeat_interleave(g, dim=1)
        mask = None
        if causal:
            i = torch.arange(sq).unsqueeze(1)
            j = torch.arange(skv).unsqueeze(0)
            mask = j <= i + (skv - sq)
        o = F.scaled_dot_product_attention(q.float(), kf, vf, attn_mask=mask, scale=scale)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), q=bits16(q), k=bits16(k), v=bits16(v),
                            o=o.numpy(), causal=np.array(causal), scale=np.array(scale, dtype=np.float64),
                            bf16=np.array(dtype == torch.bfloat16))


def paged_case():
    lens = [1, 16, 17, 95, 0, 130, 40]
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(q_heads=8, kv_heads=2, page_size=16, dtype=torch.float16,
                                                        seed=12, lens=lens)
    scale = 128 ** -0.5
    out = torch.zeros(len(lens), 8, 128)
    max_len = max(lens)
    gathered_k = torch.zeros(len(lens), 2, max_len, 128, dtype=torch.float16)
    for s, n in enumerate(lens):
        for h in range(8):
            kvh = h // 4
            if n == 0:
                continue
            krows = torch.stack([kc[int(bt[s, t // 16]), kvh, t % 16] for t in range(n)]).float()
            vrows = torch.stack([vc[int(bt[s, t // 16]), kvh, t % 16] for t in range(n)]).float()
            gathered_k[s, kvh, :n] = krows.half()
            p = torch.softmax((krows @ q[s, h].float()) * scale, dim=0)
            out[s, h] = p @ vrows
    np.savez_compressed(os.path.join(HERE, "paged_decode_f16.npz"), q=bits16(q), k_cache=bits16(kc),
                        v_cache=bits16(vc), block_table=bt.numpy(), seq_lens=sl.numpy(), o=out.numpy(),
                        gathered_k=bits16(gathered_k), scale=np.array(scale, dtype=np.float64))


def linear_cases():
    """Linear layer with bias and activation, and the two backward products of the NT form (from
    torch autograd)."""
    g = torch.Generator().manual_seed(13)
    x = (torch.randn(72, 64, generator=g) * 0.5).half()
    w = (torch.randn(88, 64, generator=g) * 0.5).half()
    bias = torch.randn(88, generator=g).half()
    dy = (torch.randn(72, 88, generator=g) * 0.5).half()
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    y = F.linear(xr, wr, bias.float())
    (y * dy.float()).sum().backward()
    np.savez_compressed(os.path.join(HERE, "linear_f16_72x88x64.npz"), x=bits16(x), w=bits16(w), bias=bits16(bias),
                        dy=bits16(dy), y_gelu=F.gelu(y.detach()).numpy(), y_silu=F.silu(y.detach()).numpy(),
                        y=y.detach().numpy(), dx=xr.grad.numpy(), dw=wr.grad.numpy())


def paged_prefill_case():
    """Append a chunk of K/V rows to a paged cache, then attend causally over everything: expected
    cache from a per-token loop, expected output from SDPA with an explicit mask per sequence."""
    lens0, chunk, hq, hkv = [50, 0, 129], 24, 4, 2
    total = [n + chunk for n in lens0]
    _, kc, vc, bt, sl = oracle.make_paged_decode_inputs(q_heads=hq, kv_heads=hkv, page_size=16, dtype=torch.bfloat16,
                                                        seed=14, lens=total)
    g = torch.Generator().manual_seed(15)
    q = (torch.randn(3, hq, chunk, 128, generator=g) * 0.5).bfloat16()
    k_new = torch.randn(3, chunk, hkv, 128, generator=g).bfloat16()
    v_new = torch.randn(3, chunk, hkv, 128, generator=g).bfloat16()
    k_after, v_after = kc.clone(), vc.clone()
    for s, n0 in enumerate(lens0):
        for t in range(chunk):
            p = n0 + t
            k_after[int(bt[s, p // 16]), :, p % 16] = k_new[s, t]
            v_after[int(bt[s, p // 16]), :, p % 16] = v_new[s, t]
    scale = 128 ** -0.5
    out = torch.zeros(3, hq, chunk, 128)
    for s, n in enumerate(total):
        kk = torch.stack([k_after[int(bt[s, t // 16]), :, t % 16] for t in range(n)], dim=1).float()
        vv = torch.stack([v_after[int(bt[s, t // 16]), :, t % 16] for t in range(n)], dim=1).float()
        kk = kk.repeat_interleave(hq // hkv, dim=0).unsqueeze(0)
        vv = vv.repeat_interleave(hq // hkv, dim=0).unsqueeze(0)
        i = torch.arange(chunk).unsqueeze(1)
        j = torch.arange(n).unsqueeze(0)
        out[s] = F.scaled_dot_product_attention(q[s:s + 1].float(), kk, vv, attn_mask=j <= i + (n - chunk), scale=scale)[0]
    np.savez_compressed(os.path.join(HERE, "paged_prefill_bf16.npz"), q=bits16(q), k_cache=bits16(kc), v_cache=bits16(vc),
                        k_new=bits16(k_new), v_new=bits16(v_new), block_table=bt.numpy(),
                        positions=np.array(lens0, dtype=np.int32), seq_lens=sl.numpy(), k_after=bits16(k_after),
                        v_after=bits16(v_after), o=out.numpy(), scale=np.array(scale, dtype=np.float64))


def attention_bwd_case():
    """Gradients from torch autograd through scaled_dot_product_attention on fp32-upcast inputs
    (grouped heads expanded with repeat_interleave, so autograd sums dK / dV over the group)."""
    sq, skv, hq, hkv, dtype = 72, 136, 4, 2, torch.bfloat16
    q, k, v = oracle.make_attention_inputs(1, hq, hkv, sq, skv, 128, dtype, seed=13, std=0.5)
    d_o = torch.randn(1, hq, sq, 128, generator=torch.Generator().manual_seed(14)).to(dtype)
    scale = 128 ** -0.5
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    i = torch.arange(sq).unsqueeze(1)
    j = torch.arange(skv).unsqueeze(0)
    mask = j <= i + (skv - sq)
    g = hq // hkv
    o = F.scaled_dot_product_attention(qf, kf.repeat_interleave(g, dim=1), vf.repeat_interleave(g, dim=1),
                                       attn_mask=mask, scale=scale)
    o.backward(d_o.float())
    np.savez_compressed(os.path.join(HERE, "attn_bwd_bf16_causal_gqa.npz"), q=bits16(q), k=bits16(k), v=bits16(v),
                        d_o=bits16(d_o), dq=qf.grad.numpy(), dk=kf.grad.numpy(), dv=vf.grad.numpy(),
                        scale=np.array(scale, dtype=np.float64))


if __name__ == "__main__":
    torch.set_num_threads(1)  # deterministic reduction order for the stored fp32 values
    gemm_case()
    attention_cases()
    paged_case()
    linear_cases()
    paged_prefill_case()
    attention_bwd_case()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
