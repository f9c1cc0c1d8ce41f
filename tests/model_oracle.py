"""CPU statement of lampa_b200.model.LSHGatedDelta for the parity tests: the same module's
weights, torch on the CPU for the host-side layers (Linear, RMS norm, GELU) with the GPU's bf16
rounding points, and the CPU checker (oracle/) in place of every library op."""
import numpy as np
import torch
import torch.nn.functional as F

from oracle import oracle


def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16)


def _linear(x_bf16: torch.Tensor, lin) -> torch.Tensor:
    """bf16 Linear as the GPU runs it: bf16 operands, wide accumulation, bf16 result."""
    y = F.linear(x_bf16.float(), lin.weight.detach().float().cpu(),
                 None if lin.bias is None else lin.bias.detach().float().cpu())
    return _bf(y)


def orderings(model, hits: np.ndarray, cu: np.ndarray) -> np.ndarray:
    ids = oracle.lsh_ids(hits, model.lsh_alpha.detach().cpu().numpy(), model.lsh_beta.detach().cpu().numpy(),
                         model.bucket_width, dim=model.coord_dim)                 # [rounds, heads, N]
    rounds, heads, n = ids.shape
    packed = np.zeros((rounds, n), np.int32)
    for h in range(heads):
        packed += ids[:, h] << h
    return np.stack([oracle.segsort(np.ascontiguousarray(packed[r]), seg=cu) for r in range(rounds)])


def mixer(attn, hs: torch.Tensor, cu: np.ndarray) -> torch.Tensor:
    """hs bf16 [n, d] in sorted order -> bf16 [n, d]."""
    n = hs.shape[0]
    H, dk, dv = attn.num_heads, attn.head_k_dim, attn.head_v_dim

    def conv(proj, cv):
        y = oracle.short_conv(_linear(hs, proj).float().numpy()[None], cv.weight.detach().float().cpu().numpy()[:, 0],
                              None if cv.bias is None else cv.bias.detach().float().cpu().numpy(), cu=cu)
        return _bf(torch.from_numpy(y[0]))

    q, k, v = conv(attn.q_proj, attn.q_conv1d), conv(attn.k_proj, attn.k_conv1d), conv(attn.v_proj, attn.v_conv1d)
    a, b, dl = (_linear(hs, p).float().numpy() for p in (attn.a_proj, attn.b_proj, attn.l_proj))
    g, beta, lam = oracle.gate_inputs(a, b, dl.reshape(n, H, attn.num_levels), attn.A_log.detach().cpu().numpy(),
                                      attn.dt_bias.detach().cpu().numpy(), attn.L.detach().cpu().numpy(), "positive")
    beta = _bf(torch.from_numpy(beta)).float().numpy()        # the library writes beta and lambda in bf16
    lam = _bf(torch.from_numpy(lam)).float().numpy()
    o, _, _ = oracle.hgdn(q.float().numpy().reshape(n, H, dk), k.float().numpy().reshape(n, H, dk),
                          v.float().numpy().reshape(n, H, dv), g, beta, lam, cu_seqlens=cu, use_l2norm=True)
    o = _bf(torch.from_numpy(o))
    gate = _linear(hs, attn.g_proj).float().numpy().reshape(n, H, dv)
    y = oracle.rmsnorm_gate(o.float().numpy(), gate, attn.o_norm.weight.detach().float().cpu().numpy(), eps=attn.o_norm.eps)
    return _linear(_bf(torch.from_numpy(y)).reshape(n, H * dv), attn.o_proj)


def forward(model, hits: torch.Tensor, cu: torch.Tensor, return_parts: bool = False):
    """hits fp32 [N, in_dim] (CPU), cu int64 [n_events + 1] -> fp32 [N, out_dim]."""
    cu_np = cu.numpy().astype(np.int64)
    perms = orderings(model, hits.numpy(), cu_np)
    x = F.linear(hits * model.feature_scale.cpu(), model.encoder.weight.detach().cpu(), model.encoder.bias.detach().cpu())
    parts, streams = [], []
    for b, blk in enumerate(model.blocks):
        streams.append(x.clone())
        d = x.shape[1]
        perm = perms[b % model.rounds]
        h = _bf(F.rms_norm(x, (d,), blk.attn_norm_weight.detach().cpu(), blk.eps))
        hs = torch.from_numpy(oracle.permute_rows(h.float().numpy(), perm, seg=cu_np))
        o = mixer(blk.attn, _bf(hs), cu_np)
        back = oracle.permute_rows(o.float().numpy(), oracle.invert_perm(perm, seg=cu_np), seg=cu_np)
        mix = torch.from_numpy(back)
        parts.append((float(mix.norm()), float(x.norm())))
        x = x + mix
        h = _bf(F.rms_norm(x, (d,), blk.mlp_norm_weight.detach().cpu(), blk.eps))
        x = x + _linear(_bf(F.gelu(_linear(h, blk.mlp_up).float())), blk.mlp_down).float()
    y = F.linear(x, model.head.weight.detach().cpu(), model.head.bias.detach().cpu())
    streams.append(x.clone())
    return (y, perms, parts, streams) if return_parts else y
