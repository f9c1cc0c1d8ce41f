"""Generate the golden fixtures in this directory from the reference's own code.

Run once in a container where the reference checkout is mounted:

    python tests/golden/gen_golden.py --reference /path/to/Lampa

It executes the reference's pure-PyTorch CPU statements of the path
(models/hattention/recurrent.py::hattention_recurrent,
models/hattention/base.py::hattention_materialized_dplr helpers,
models/baselines/hmamba.py::LSHOrdering / E2LSH / lsh_mapping,
models/model_utils/hash_utils.py::invert_permutation / batched_index_select,
models/attention/hept.py::sort_to_buckets / unsort_from_buckets / get_geo_shift,
models/model_utils/hash_utils.py::pad_to_multiple / get_regions / quantile_partition /
E2LSH / lsh_mapping, and the layer statements listed in gen_layer) on seeded
inputs and stores inputs + outputs as small .npz files.  Nothing from the
reference is copied; only numbers it produced are stored.
"""
from __future__ import annotations

import argparse
import ast
import importlib
import importlib.util
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


def load_hattention(ref: str):
    """Register a synthetic package over models/hattention and import base + recurrent."""
    pkg_dir = os.path.join(ref, "models", "hattention")
    pkg = types.ModuleType("_ref_hattention")
    pkg.__path__ = [pkg_dir]
    sys.modules["_ref_hattention"] = pkg
    mods = {}
    for name in ("base", "recurrent"):
        spec = importlib.util.spec_from_file_location(
            f"_ref_hattention.{name}", os.path.join(pkg_dir, f"{name}.py"))
        m = importlib.util.module_from_spec(spec)
        sys.modules[f"_ref_hattention.{name}"] = m
        spec.loader.exec_module(m)
        mods[name] = m
    return mods["base"], mods["recurrent"]


def load_defs(path: str, names, extra=None):
    """Execute only the named top-level defs/classes of a file (its imports may be unavailable)."""
    tree = ast.parse(open(path).read())
    keep = [n for n in tree.body
            if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    scope = {"torch": torch, "nn": nn}
    scope.update(extra or {})
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), scope)
    return scope


def gdn_inputs(seed, T, H, K, V, L=None, g_shift=2.0):
    gen = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(T, H, K, generator=gen), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(T, H, K, generator=gen), dim=-1)
    v = torch.randn(T, H, V, generator=gen)
    beta = torch.sigmoid(torch.randn(T, H, generator=gen))
    g = -torch.nn.functional.softplus(torch.randn(T, H, generator=gen) + g_shift)
    lam = None if L is None else torch.nn.functional.softplus(torch.randn(T, H, L, generator=gen))
    return q, k, v, beta, g, lam


def gen_geo(ref: str):
    """Region shift of the HEPT keys: the statements of prepare_input
    (models/hattention/modeling_gated_deltaproduct.py:1210-1222) and of HEPTAttention.forward
    up to the positions (models/attention/hept.py:118-138), run with the reference's functions."""
    einops = __import__("einops")
    hu = load_defs(os.path.join(ref, "models", "model_utils", "hash_utils.py"),
                   {"pad_to_multiple", "get_regions", "quantile_partition", "E2LSH", "lsh_mapping", "uniform"},
                   extra={"rearrange": einops.rearrange, "F": torch.nn.functional})
    hp = load_defs(os.path.join(ref, "models", "attention", "hept.py"), {"get_geo_shift"},
                   extra={"rearrange": einops.rearrange, "List": list})
    rearrange = einops.rearrange
    raw, block, heads, rounds, dim, num_regions = 1090, 100, 4, 3, 8, 40
    gen = torch.Generator().manual_seed(4242)
    eta = torch.randn(raw, generator=gen) * 1.5
    phi = (torch.rand(raw, generator=gen) * 2 - 1) * np.pi
    coords_raw = torch.stack([eta, phi], -1)
    q_raw = torch.randn(heads, raw, dim, generator=gen)
    k_raw = torch.randn(heads, raw, dim, generator=gen)
    torch.manual_seed(11)
    regions = hu["get_regions"](num_regions, rounds, heads)              # [c, a, h]
    e2lsh = hu["E2LSH"](n_hashes=rounds, n_heads=heads, dim=dim)
    with torch.no_grad():
        coords = hu["pad_to_multiple"](coords_raw, block, dims=0, value=float("inf"))
        sorted_eta = torch.argsort(coords[..., 0], dim=-1)
        sorted_phi = torch.argsort(coords[..., 1], dim=-1)
        regions_h = rearrange(regions, "c a h -> a (c h)")
        reg_eta = hu["quantile_partition"](sorted_eta, regions_h[0][:, None])
        reg_phi = hu["quantile_partition"](sorted_phi, regions_h[1][:, None])
        n = coords.shape[0]
        q_hat = torch.zeros(heads, n, dim); q_hat[:, :raw] = q_raw
        k_hat = torch.zeros(heads, n, dim); k_hat[:, :raw] = k_raw
        qh, kh, hs = hu["lsh_mapping"](e2lsh, q_hat, k_hat)
        hs = rearrange(hs, "c h d -> (c h) d")
        qh[..., raw:] = float("inf")
        kh[..., raw:] = float("inf")
        q_shift, k_shift = hp["get_geo_shift"](regions_h, hs, [reg_eta, reg_phi], rounds)
        q_keys = qh + q_shift
        k_keys = kh + k_shift
        q_pos = q_keys.argsort(dim=-1)
        k_pos = k_keys.argsort(dim=-1)
    np.savez_compressed(
        os.path.join(HERE, "geo_shift_N1090_R12.npz"),
        coords=coords_raw.numpy(), q_hat=q_hat.numpy(), k_hat=k_hat.numpy(), regions=regions.numpy(),
        alpha=e2lsh.alpha.detach().numpy(), beta=e2lsh.beta.detach().numpy(),
        raw_size=np.int64(raw), block_size=np.int64(block),
        sorted_eta=sorted_eta.numpy(), sorted_phi=sorted_phi.numpy(),
        reg_eta=reg_eta.numpy(), reg_phi=reg_phi.numpy(), hash_shift=hs.numpy(),
        q_hashed=qh.numpy(), k_hashed=kh.numpy(), q_shift=q_shift.numpy(), k_shift=k_shift.numpy(),
        q_keys=q_keys.numpy(), k_keys=k_keys.numpy(), q_pos=q_pos.numpy(), k_pos=k_pos.numpy())
    print("geo ok", tuple(reg_eta.shape), tuple(q_pos.shape), float(hs.max()))


def gen_layer(ref: str):
    """Producers / consumers of the op inside one HGatedDeltaNet layer, from the reference's own
    pure-PyTorch statements: compute_lambda (models/hattention/modeling_h_gated_deltanet.py:151-166),
    the g / beta expressions of HGatedDeltaNet.forward (429-430, restated here since they are
    inline), ShortConvolution's parameters and its documented equivalent
    `_conv_forward(x, weight, bias)[..., :T]` + SiLU (models/hattention/short_convolution.py:528-573,
    650-654), the cache statements (617-626, 700-703), and rms_norm_ref followed by the swish gate of
    the fused kernel (models/hattention/fused_norm.py:1306-1327, 99-107)."""
    import warnings
    from typing import Optional, Tuple
    import torch.nn.functional as F
    einops = __import__("einops")
    hd = os.path.join(ref, "models", "hattention")
    ml = load_defs(os.path.join(hd, "modeling_h_gated_deltanet.py"), {"compute_lambda"},
                   extra={"warnings": warnings, "click": __import__("click"), "Optional": Optional})
    sc = load_defs(os.path.join(hd, "short_convolution.py"), {"ShortConvolution"},
                   extra={"warnings": warnings, "Optional": Optional, "Tuple": Tuple, "rearrange": einops.rearrange,
                          "causal_conv1d_fn": None, "causal_conv1d_update_cuda": None})
    fn = load_defs(os.path.join(hd, "fused_norm.py"), {"rms_norm_ref"}, extra={"F": F})
    gen = torch.Generator().manual_seed(777)
    B, T, H, Lv, D, W, Dv = 2, 70, 3, 9, 48, 4, 32
    a = torch.randn(B, T, H, generator=gen)
    b = torch.randn(B, T, H, generator=gen)
    dl = torch.randn(B, T, H, Lv, generator=gen) * 2
    A_log = torch.log(torch.empty(H).uniform_(0, 16, generator=gen))
    dt_bias = torch.randn(H, generator=gen)
    Lp = 1 + 0.3 * torch.randn(H, Lv, generator=gen)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        lam = {m: ml["compute_lambda"](Lp[None, None], dl, m) for m in ("positive", "bounded", None)}
    g = -A_log.float().exp() * F.softplus(a.float() + dt_bias)
    beta = b.sigmoid()
    torch.manual_seed(3)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        conv = sc["ShortConvolution"](hidden_size=D, kernel_size=W, bias=True, activation="silu", use_fast_conv1d=False)
    x = torch.randn(B, T, D, generator=gen)
    res = torch.randn(B, T, D, generator=gen)
    with torch.no_grad():
        y = F.silu(conv._conv_forward(x.transpose(1, 2), conv.weight, conv.bias)[..., :T]).transpose(1, 2) + res
        cache = torch.zeros(B, D, W)
        cache[:, :, -min(W, T):].copy_(x[..., -min(W, T):, :].transpose(1, 2))
        # packed: two sequences of 31 and 39 tokens taken from batch row 0
        cu = [0, 31, 70]
        yv = torch.cat([F.silu(conv._conv_forward(x[0:1, s:e].transpose(1, 2), conv.weight, conv.bias)[..., :e - s]).transpose(1, 2)
                        for s, e in zip(cu[:-1], cu[1:])], 1)
        # decode step on the cache: roll, insert, weighted sum
        xs = torch.randn(B, 1, D, generator=gen)
        c2 = cache.roll(shifts=-1, dims=-1)
        c2[:, :, -1] = xs[:, 0]
        ys = F.silu(torch.sum(c2 * conv.weight[:, 0], dim=-1) + conv.bias)[:, None]
        xo = torch.randn(B, T, H, Dv, generator=gen)
        go = torch.randn(B, T, H, Dv, generator=gen)
        wn = 1 + 0.2 * torch.randn(Dv, generator=gen)
        yn = fn["rms_norm_ref"](xo, wn, None, eps=1e-5, upcast=True)
        yn = yn * go * torch.sigmoid(go)
    np.savez_compressed(
        os.path.join(HERE, "layer_ops.npz"),
        a=a.numpy(), b=b.numpy(), dl=dl.numpy(), A_log=A_log.numpy(), dt_bias=dt_bias.numpy(), L=Lp.numpy(),
        g=g.numpy(), beta=beta.numpy(), lam_positive=lam["positive"].numpy(), lam_bounded=lam["bounded"].numpy(),
        lam_default=lam[None].numpy(),
        conv_w=conv.weight.detach().numpy(), conv_b=conv.bias.detach().numpy(), x=x.numpy(), res=res.numpy(),
        y=y.numpy(), cache=cache.numpy(), cu=np.array(cu, np.int64), y_packed=yv.numpy(),
        x_step=xs.numpy(), y_step=ys.numpy(), cache_step=c2.numpy(),
        norm_x=xo.numpy(), norm_g=go.numpy(), norm_w=wn.numpy(), norm_y=yn.numpy())
    print("layer ok", tuple(y.shape), float(y.abs().max()), float(yn.abs().max()))


def gen_hept(ref: str):
    """Bucketed attention of the HEPT layer: prep_qk, sort_to_buckets, qkv_res, unsort_from_buckets
    and the combination over rounds (models/attention/hept.py:9-33, 55-63, 141-151), run with the
    reference's functions on seeded inputs with random bucket orders."""
    einops = __import__("einops")
    hu = load_defs(os.path.join(ref, "models", "model_utils", "hash_utils.py"),
                   {"batched_index_select", "invert_permutation"}, extra={"rearrange": einops.rearrange})
    hp = load_defs(os.path.join(ref, "models", "attention", "hept.py"),
                   {"sort_to_buckets", "unsort_from_buckets", "qkv_res", "prep_qk"},
                   extra={"rearrange": einops.rearrange, "List": list,
                          "batched_index_select": hu["batched_index_select"]})
    rearrange = einops.rearrange
    raw, n, block, heads, rounds, d, cd, nw = 570, 600, 100, 3, 3, 12, 6, 4
    gen = torch.Generator().manual_seed(777)
    query = torch.randn(n, heads, d, generator=gen) * 0.7
    key = query + 0.4 * torch.randn(n, heads, d, generator=gen)
    value = torch.randn(n, heads, d, generator=gen)
    coords = torch.randn(n, cd, generator=gen) * 0.5
    coords[raw:] = 0.0
    w = torch.randn(heads, d, cd - 1, nw, generator=gen) * 0.3 - 0.6
    q_pos = torch.stack([torch.stack([torch.randperm(n, generator=gen) for _ in range(heads)]) for _ in range(rounds)])
    k_pos = torch.stack([torch.stack([torch.randperm(n, generator=gen) for _ in range(heads)]) for _ in range(rounds)])
    with torch.no_grad():
        q_hat, k_hat = hp["prep_qk"](query, key, w, coords)
        q_hat = rearrange(q_hat, "n h d -> h n d").contiguous()
        k_hat = rearrange(k_hat, "n h d -> h n d").contiguous()
        v = rearrange(value, "n h d -> h n d").contiguous()
        q_hat[:, raw:] = 0.0
        k_hat[:, raw:] = 0.0
        v[:, raw:] = 0.0
        s_query = hp["sort_to_buckets"](q_hat, q_pos, block)
        s_key = hp["sort_to_buckets"](k_hat, k_pos, block)
        s_value = hp["sort_to_buckets"](v, k_pos, block)
        denom, so = hp["qkv_res"](s_query, s_key, s_value)
        q_rev = hu["invert_permutation"](q_pos)
        o = hp["unsort_from_buckets"](so, q_rev)
        logits = hp["unsort_from_buckets"](denom, q_rev)
        out = o.sum(dim=0) / logits.sum(dim=0)
    np.savez_compressed(
        os.path.join(HERE, "hept_bucket_attn.npz"),
        query=query.numpy(), key=key.numpy(), value=value.numpy(), coords=coords.numpy(), w=w.numpy(),
        q_pos=q_pos.numpy(), k_pos=k_pos.numpy(), raw_size=np.int64(raw), block_size=np.int64(block),
        q_hat=q_hat.numpy(), k_hat=k_hat.numpy(), v=v.numpy(), denom=denom.numpy(), so=so.numpy(),
        o=o.numpy(), logits=logits.numpy(), out=out.numpy())
    print("hept ok", tuple(so.shape), tuple(out.shape), float(denom.min()), float(denom.max()))


def gen_minimal(ref: str):
    """The reference's own chunkwise statement of the hierarchical rule, hgdn_minimal
    (models/hattention/hssd_minimal.py:462-493), at T = 4096 (64 chunks: two blocks of 32, one
    cross-block level).  Its level table comes from make_levels_matrix (models/hattention/base.py:
    101-161), a Python double loop over T x T (and over 16384 x 16384 through its cache) that
    cannot finish at this length; it is replaced here by the same table built with
    bit_length(t XOR s), the closed form the reference's own get_level_index_weak reproduces for
    every pair of levels_weak_130.npz.  Everything else is the reference's code, in fp32."""
    pkg_dir = os.path.join(ref, "models", "hattention")
    if "_ref_hattention" not in sys.modules:
        load_hattention(ref)
    base = sys.modules["_ref_hattention.base"]

    def levels_closed_form(length, base, htype, dtype, device, default=-1, clamp_min=None, file_name=None,
                           cached_length=None):
        t = np.arange(length)[:, None]
        s_ = np.arange(length)[None, :]
        x = t ^ s_
        bl = np.zeros_like(x)
        nz = x > 0
        bl[nz] = np.floor(np.log2(x[nz])).astype(np.int64) + 1
        lv = np.where(s_ <= t, bl, default)
        out = torch.from_numpy(lv.astype(np.int64)).to(dtype=dtype, device=device)
        return out if clamp_min is None else torch.clamp(out, min=clamp_min)

    # the closed form against the reference's own level function on a prefix
    chk = levels_closed_form(130, 2, base.HType.WEAK, torch.int64, "cpu")
    for t in range(130):
        for s_ in range(t):
            assert int(chk[t, s_]) == base.get_level_index_weak(t, s_, 2)
    for name in ("fla_utils", "fla_op", "cumsum", "hssd_minimal"):
        if f"_ref_hattention.{name}" in sys.modules:
            continue
        spec = importlib.util.spec_from_file_location(f"_ref_hattention.{name}", os.path.join(pkg_dir, f"{name}.py"))
        m = importlib.util.module_from_spec(spec)
        sys.modules[f"_ref_hattention.{name}"] = m
        try:
            spec.loader.exec_module(m)
        except Exception as e:                      # helper modules that need a GPU stack: only hssd_minimal must load
            if name == "hssd_minimal":
                raise
            print("note:", name, "not importable here:", type(e).__name__)
    mini = sys.modules["_ref_hattention.hssd_minimal"]
    mini.make_levels_matrix = levels_closed_form
    T, H, K, V = 4096, 2, 32, 32
    Lv = 7 + 6
    q, k, v, beta, g, lam = gdn_inputs(104, T, H, K, V, Lv, -4.0)     # the test redraws these from the seed
    scale = K ** -0.5
    with torch.no_grad():
        o = mini.hgdn_minimal(Q=(q * scale)[None], K=k[None], V=v[None], B=beta[None], G=g[None], L=(lam / scale)[None],
                              level_base=2, htype=base.HType.WEAK, block_len=64)
    np.savez_compressed(os.path.join(HERE, "hgdn_minimal_T4096_H2_K32_V32_L13.npz"),
                        seed=np.int64(104), g_shift=np.float32(-4.0), shape=np.array([T, H, K, V, Lv]),
                        input_sums=np.array([float(x.double().sum()) for x in (q, k, v, beta, g, lam)]),
                        o_hier=o[0].numpy())
    print("hgdn_minimal ok", tuple(o.shape), float(o.abs().max()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", default="", help="'geo' / 'layer' / 'hept' / 'minimal': write only that fixture")
    args = ap.parse_args()
    ref = args.reference
    torch.set_num_threads(8)
    if args.only in ("", "geo"):
        gen_geo(ref)
    if args.only in ("", "hept"):
        gen_hept(args.reference)
    if args.only in ("", "layer"):
        gen_layer(ref)
    if args.only in ("", "minimal"):
        gen_minimal(ref)
    if args.only:
        return
    base, recurrent = load_hattention(ref)

    # ---- hierarchical + plain gated delta, reference token recurrence -------------
    cases = [
        ("hgdn_T200_H2_K16_V32_L9", 101, 200, 2, 16, 32, 9, 2.0),
        ("hgdn_T320_H2_K32_V32_L10", 102, 320, 2, 32, 32, 10, -3.0),
        ("hgdn_T256_H1_K64_V64_L9", 103, 256, 1, 64, 64, 9, -4.0),
    ]
    for name, seed, T, H, K, V, L, gs in cases:
        q, k, v, beta, g, lam = gdn_inputs(seed, T, H, K, V, L, gs)
        scale = K ** -0.5
        # API layer semantics: Q = l2norm(q)*scale, L = lambda/scale (inputs are already unit-norm)
        o, S = recurrent.hattention_recurrent(
            Q=(q * scale)[None], K=k[None], V=v[None], A=torch.exp(g)[None], B=beta[None],
            L=(lam / scale)[None], base=2, htype=base.HType.WEAK, hstruct=base.HStruct.GDELTA)
        o1, S1 = recurrent.hattention_recurrent(
            Q=(q * scale)[None], K=k[None], V=v[None], A=torch.exp(g)[None], B=beta[None],
            L=torch.ones_like(lam)[None], base=2, htype=base.HType.WEAK, hstruct=base.HStruct.GDELTA)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            q=q.numpy(), k=k.numpy(), v=v.numpy(), beta=beta.numpy(), g=g.numpy(), lam=lam.numpy(),
            o_hier=o[0].numpy(), states_hier=S.states[0].numpy(), counts_hier=S.counts.numpy(),
            o_plain=o1[0].numpy(), final_plain=S1.states[0].sum(-1).numpy(), scale=np.float32(scale))
        print(name, "ok", float(o.abs().max()))

    # level function of the reference vs bit_length(t ^ s)
    lv = np.array([[base.get_level_index_weak(t, s, 2) if s < t else 0 for s in range(130)]
                   for t in range(130)], np.int32)
    np.savez_compressed(os.path.join(HERE, "levels_weak_130.npz"), levels=lv)

    # ---- LSH ordering ------------------------------------------------------------
    hm = load_defs(os.path.join(ref, "models", "baselines", "hmamba.py"),
                   {"lsh_mapping", "E2LSH", "LSHOrdering"})
    sys.path.insert(0, os.path.join(ref, "models", "model_utils"))
    hu = load_defs(os.path.join(ref, "models", "model_utils", "hash_utils.py"),
                   {"invert_permutation", "batched_index_select"},
                   extra={"rearrange": __import__("einops").rearrange})
    hp = load_defs(os.path.join(ref, "models", "attention", "hept.py"),
                   {"sort_to_buckets", "unsort_from_buckets"},
                   extra={"rearrange": __import__("einops").rearrange,
                          "batched_index_select": hu["batched_index_select"]})

    gen = torch.Generator().manual_seed(2025)
    Bn, Ln, D, C = 2, 1500, 8, 6
    layer = torch.randint(0, 10, (Bn, Ln), generator=gen).float()
    r = 30 + layer * (970.0 / 9)
    phi = (torch.rand(Bn, Ln, generator=gen) * 2 - 1) * np.pi
    z = (torch.rand(Bn, Ln, generator=gen) * 2 - 1) * 3000
    coords = torch.stack([r * torch.cos(phi), r * torch.sin(phi), z, r, phi, torch.asinh(z / r)], -1)
    points = torch.randn(Bn, Ln, D, generator=gen)
    torch.manual_seed(7)
    ordering = hm["LSHOrdering"](C, num_hashes=3)
    ordered, idx = ordering(points, coords)
    flat = coords.reshape(Bn * Ln, C).unsqueeze(0)
    proj = ordering.e2lsh(flat)                      # [n_hashes, N, n_heads=1]
    inv = hu["invert_permutation"](idx)
    buckets = hp["sort_to_buckets"](points, idx[None], 100)
    unsorted = hp["unsort_from_buckets"](buckets, inv[None])
    np.savez_compressed(
        os.path.join(HERE, "lsh_ordering_B2_L1500.npz"),
        coords=coords.numpy(), points=points.numpy(), alpha=ordering.e2lsh.alpha.detach().numpy(),
        beta=ordering.e2lsh.beta.detach().numpy(), proj=proj.numpy(), indices=idx.numpy(),
        ordered=ordered.numpy(), inverse=inv.numpy(), buckets=buckets.numpy(),
        unsorted=unsorted.numpy())
    print("lsh ok", idx.shape, buckets.shape, bool((unsorted[0] == points).all()))


if __name__ == "__main__":
    main()
