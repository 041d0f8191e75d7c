"""The Gozatar parts and the whole decoder against the plain implementation in ``plain/gozatar_plain.py``.

Each mechanism alone (kernel against its formula), then small models with random weights under every way of cutting
the work: whole prompts, token-by-token decoding, portions down to two tokens, batches of unequal requests, slots
and pages used again, long decoding with a window that passes over decoded tokens, greedy generation through
``Engine.generate``, and the trace program. Where random weights would hide a fault (one key among many, the window's
edge), the weights are made so that one key dominates the attention.
"""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import tiny
import traces
from plain import gozatar_plain as G
from plain.llama_plain import read_model_folder
from spissa_b200 import Engine, SamplingParams
from spissa_b200.config import config_from_dict
from spissa_b200.weights import write_random_model, write_safetensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def left(heads, kv, dim, vdim, conv=None, rot=None, base=10000.0, window=None, scale=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale or 1.0 / math.sqrt(dim))
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    if window:
        m["mask"] = dict(size=window)
    return m


def par(l, heads, dim, vdim, tau, ls=1.0, rs=1.0, rank=None):
    r = dict(heads=heads, dim=dim, vdim=vdim, tau=tau)
    if rank:
        r["rank"] = rank
    return dict(type="parallel", mixer=dict(left=l, right=r, left_scale=ls, right_scale=rs))


def moe(experts, top, ff, limit, groups=None, shared=None):
    r = dict(experts=experts, top=top)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=r, shared=dict(ff=shared[0], limit=shared[1]) if shared else None)


def dense(ff):
    return dict(kind="dense", ff=ff)


def model(width, vocab, layers, mlps, streams=None, eps=1e-5):
    out = dict(architecture="Gozatar", vocab=vocab, width=width, norm=dict(eps=eps),
               layers=[dict(l, mlp=f) for l, f in zip(layers, mlps)])
    if streams:
        out["streams"] = streams
    return out


# sizes that differ from one another everywhere: grouped, multi-head and single-kv-head attention; key and value sizes
# equal or not; convolutions of 4, 2, 3, 5 taps, of one tap (a weight per channel) or none; rotation over a part of the dims, all, or none; windows below and
# above a page, or none; one, three, four streams or plain residual sums; experts in groups of 2, 3, 1 or ungrouped,
# with and without a shared expert; layers without a feed-forward
CONFIGS = {
    "a": model(64, 200, [par(left(4, 2, 16, 16, conv=4, rot=8, window=20), 2, 8, 16, 4.0, 0.7, 0.4),
                         par(left(2, 1, 32, 32, conv=2, rot=32, base=100.0, window=7), 3, 16, 8, 16.0, 1.2, 0.9, rank=3),
                         par(left(2, 2, 16, 48, conv=3, rot=4, window=70), 1, 8, 24, 2.0, 0.5, 1.5)],
               [moe(8, 2, 24, 1.5, groups=(4, 2), shared=(40, 3.0)), dense(80), None], streams=3),
    "b": model(96, 333, [par(left(3, 3, 12, 20, conv=2, rot=12, window=70), 1, 16, 40, 1.0, 1.0, 1.0),
                         par(left(6, 2, 16, 16, conv=1, rot=6, base=500.0, window=130), 2, 8, 8, 8.0, 0.3, 0.6)],
               [moe(6, 3, 32, 0.8), moe(9, 3, 16, 2.5, groups=(3, 1), shared=(24, 1.0))], streams=1, eps=1e-3),
    "c": model(48, 150, [par(left(2, 1, 32, 32), 3, 8, 8, 30.0, 0.9, 0.2),
                         par(left(1, 1, 16, 8, conv=3, window=33), 2, 4, 12, 0.7, 1.0, 1.0)],
               [dense(96), moe(4, 2, 20, 1.0, groups=(4, 2))], streams=None),
    # nothing a multiple of four: the paths without wide loads, an odd head size of which four dims turn
    "d": model(50, 97, [par(left(2, 1, 7, 9, conv=3, rot=4, window=9), 2, 5, 7, 3.0, 0.8, 1.1, rank=3),
                        par(left(3, 3, 10, 6, conv=5, rot=10, window=65), 1, 6, 10, 5.0, 1.0, 0.5)],
               [moe(4, 1, 10, 2.0, groups=(2, 1), shared=(14, 0.5)), dense(30)], streams=4),
}
INIT = {"a": dict(seed=5, std=0.08, norm_std=0.2), "b": dict(seed=9, std=0.06, norm_std=0.1),
        "c": dict(seed=13, std=0.1, norm_std=0.3), "d": dict(seed=17, std=0.12, norm_std=0.2)}


def make(cfg, folder, seed, std, norm_std, patch=None):
    write_random_model(config_from_dict(cfg), folder, seed=seed, std=std, norm_std=norm_std)
    pcfg, w = read_model_folder(folder)
    # the random-weights mode gives every tap one value and the small tables values close to one another: spread them, so
    # that a tap taken from the wrong token, a swapped coefficient or a correction left out shows
    g = torch.Generator().manual_seed(seed)
    for name in sorted(w):
        last = name.split(".")[-1]
        if last == "conv":
            w[name] = torch.randn(w[name].shape, generator=g).to(w[name].dtype)
        elif ".hc" in name and last == "mix":
            w[name] = (torch.eye(w[name].shape[0]) + 0.4 * torch.randn(w[name].shape, generator=g)).to(w[name].dtype)
        elif ".hc" in name:
            w[name] = (0.3 + torch.rand(w[name].shape, generator=g)).to(w[name].dtype)
        elif last == "correction":
            w[name] = (0.5 * torch.randn(w[name].shape, generator=g)).to(w[name].dtype)
        elif last == "router":
            w[name] = (4.0 * w[name].float()).to(w[name].dtype)
        elif name.endswith("a2.b"):
            w[name] = (2.0 * torch.randn(w[name].shape, generator=g) + 1.0).to(w[name].dtype)
        elif last in ("a1", "a2"):
            w[name] = (6.0 * w[name].float()).to(w[name].dtype)
    if patch:
        patch(w)
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    return read_model_folder(folder)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"gz_{name}")
        pcfg, w = make(cfg, folder, **INIT[name])
        out[name] = SimpleNamespace(folder=str(folder), cfg=pcfg, w=w, vocab=cfg["vocab"])
    return out


def worst(got, ref):
    return float((got.double().cpu() - ref.double()).abs().max() / ref.abs().max())


def logits_of(m, toks):
    return G.forward(m.cfg, m.w, toks)


# ---------------------------------------------------------------------------------------------- each mechanism alone
def _step(lengths, slots=None, before=None):
    """The device arrays a kernel wants of a step with sequences of these lengths (``before``: tokens already cached)."""
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    seq = [b for b, n in enumerate(lengths) for _ in range(n)]
    before = before or [0] * len(lengths)
    pos = [before[b] + i for b, n in enumerate(lengths) for i in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(seq_start=i32(starts), seq_slot=i32(slots or list(range(len(lengths)))), token_seq=i32(seq),
                           positions=i32(pos), n_seqs=len(lengths), all_single=all(n == 1 for n in lengths),
                           max_new=max(lengths), host=dict(new_counts=list(lengths)))


@pytest.mark.parametrize("S,W,out_dtype", [(1, 40, torch.float32), (3, 50, torch.float32), (4, 1030, torch.bfloat16), (8, 16, torch.float32)])
def test_streams_take_a_sublayer_in_and_the_norm_reads_their_mix(S, W, out_dtype):
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(S * W)
    T = 13
    x = 3 * torch.randn(T, S, W, generator=g) + 2.0
    y = torch.randn(T, W, generator=g)
    mix, oc, ic = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    wn = torch.randn(W, generator=g)
    X = x.double().permute(1, 0, 2)
    new = torch.einsum("sr,stw->rtw", mix.double(), X) + oc.double()[:, None, None] * y.double()[None]
    ref = G.layer_norm(torch.einsum("s,stw->tw", ic.double(), new), wn.double(), 1e-3)
    xd, yd = x.reshape(T, S * W).to(DEV).contiguous(), y.to(DEV)
    out = torch.empty(T, W, dtype=out_dtype, device=DEV)
    K.streams_norm(xd, S, W, out=out, weight=wn.to(DEV), eps=1e-3, y=yd, mix=mix.to(DEV), out_coef=oc.to(DEV), in_coef=ic.to(DEV))
    tol = 1e-5 if out_dtype == torch.float32 else 6e-3
    assert worst(out, ref) <= tol
    assert worst(xd.view(T, S, W).permute(1, 0, 2), new) <= 1e-6
    assert float(yd.abs().max()) == 0.0                          # left zeroed for the next sublayer to add into
    # the norm alone over gathered rows, of the plain sum of the streams
    rows = torch.tensor([5, 0, 12], dtype=torch.int32, device=DEV)
    some = torch.empty(3, W, dtype=torch.float32, device=DEV)
    K.streams_norm(xd, S, W, out=some, weight=wn.to(DEV), eps=1e-3, rows=rows)
    assert worst(some, G.layer_norm(new.sum(0)[rows.long().cpu()], wn.double(), 1e-3)) <= 1e-5
    # the update alone
    K.streams_norm(xd, S, W, y=torch.ones(T, W, device=DEV), mix=mix.to(DEV), out_coef=oc.to(DEV))
    again = torch.einsum("sr,stw->rtw", mix.double(), new) + oc.double()[:, None, None]
    assert worst(xd.view(T, S, W).permute(1, 0, 2), again) <= 1e-6


@pytest.mark.parametrize("nh,nkv,d,vd,taps,rd,unit", [(4, 2, 16, 16, 4, 8, True), (2, 1, 7, 9, 3, 4, True), (3, 3, 12, 20, 1, 12, False),
                                                      (1, 1, 40, 8, 8, 0, True), (2, 2, 130, 6, 2, 130, True)])
def test_convolution_rotation_and_unit_rms_across_steps_and_slots(nh, nkv, d, vd, taps, rd, unit):
    """Three sequences in scattered slots and pages, cut into steps of unequal portions (one of them a token at a
    time): what lands in the pages and in q must be what the plain functions give on the whole sequences."""
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(nh * d + taps)
    C = (nh + nkv) * d + nkv * vd
    lengths, slots, eps, base = [70, 9, 131], [2, 0, 3], 1e-4, 300.0
    u = [torch.randn(n, C, generator=g) for n in lengths]
    conv = torch.randn(C, taps, generator=g) if taps > 1 else None
    inv_freq = torch.tensor([base ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float32) if rd else None
    ps, n_pages = 64, 12
    pages = [[7, 3], [5], [1, 9, 4]]
    table = torch.zeros(3, 3, dtype=torch.int32)
    for b, p in enumerate(pages):
        table[b, :len(p)] = torch.tensor(p)
    kpool = torch.zeros(n_pages, nkv, ps, d, device=DEV)
    vpool = torch.zeros(n_pages, nkv, ps, vd, device=DEV)
    state = torch.zeros(4, max(taps - 1, 1), C, device=DEV)
    cuts = [[5, 1, 1, 63, 0], [2, 1, 1, 5, 0], [64, 1, 1, 1, 64]]                      # per sequence, per step
    at = [0, 0, 0]
    q_rows = [[], [], []]
    for s in range(5):
        live = [b for b in range(3) if cuts[b][s] > 0]
        ns = [cuts[b][s] for b in live]
        step = _step(ns, [slots[b] for b in live], [at[b] for b in live])
        meta = SimpleNamespace(token_seq=step.token_seq, positions=step.positions, page_size=ps,
                               seq_slot=torch.tensor(live, dtype=torch.int32, device=DEV), page_table=table.to(DEV))
        qkv = torch.cat([u[b][at[b]:at[b] + n] for b, n in zip(live, ns)]).to(DEV)
        q = torch.empty(qkv.shape[0], nh * d, device=DEV)
        K.conv_qk_store(qkv, conv.to(DEV) if conv is not None else None, taps, state if taps > 1 else None, q, kpool, vpool,
                        meta, step, inv_freq.to(DEV) if rd else None, nh, nkv, d, vd, rd, eps, v_scale=0.5, unit_rms=unit)
        o = 0
        for b, n in zip(live, ns):
            q_rows[b].append(q[o:o + n].cpu())
            o += n
            at[b] += n
    for b, n in enumerate(lengths):
        full = G.short_conv(u[b].double(), conv.double()) if conv is not None else u[b].double()
        rq = full[:, :nh * d].view(n, nh, d)
        rk = full[:, nh * d:(nh + nkv) * d].view(n, nkv, d)
        rv = full[:, (nh + nkv) * d:].view(n, nkv, vd) * 0.5
        rq, rk = G.rotate_half(rq, rd, base), G.rotate_half(rk, rd, base)
        if unit:
            rq, rk = G.unit_rms(rq, eps), G.unit_rms(rk, eps)
        assert worst(torch.cat(q_rows[b]), rq.reshape(n, -1)) <= 3e-6, b
        got_k = torch.cat([kpool[p].permute(1, 0, 2) for p in pages[b]])[:n].cpu()
        got_v = torch.cat([vpool[p].permute(1, 0, 2) for p in pages[b]])[:n].cpu()
        assert worst(got_k, rk) <= 3e-6 and worst(got_v, rv) <= 3e-6, b
        if taps > 1:
            assert torch.equal(state[slots[b]].cpu(), u[b][n - (taps - 1):])           # the last inputs, oldest first


@pytest.mark.parametrize("H,d,vd,rank,tau", [(2, 8, 16, 3, 4.0), (1, 16, 40, 16, 1.0), (3, 5, 7, 2, 0.5), (2, 64, 64, 8, 16.0),
                                             (1, 130, 33, 4, 2.0)])
def test_gated_linear_attention_whole_in_portions_and_token_by_token(H, d, vd, rank, tau):
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(H * d + vd)
    W, eps, scale = 24, 1e-4, 0.6
    lengths, slots = [150, 37], [1, 3]
    w = {"q": torch.randn(H * d, W, generator=g) * 0.3, "k": torch.randn(H * d, W, generator=g) * 0.3,
         "v": torch.randn(H * vd, W, generator=g) * 0.3, "g": torch.randn(H * vd, W, generator=g) * 0.3,
         "a1": torch.randn(rank, W, generator=g), "a2": torch.randn(H * d, rank, generator=g),
         "a2.b": 2 * torch.randn(H * d, generator=g), "norm": torch.randn(vd, generator=g), "o": torch.eye(H * vd)}
    wd = {k: v.double() for k, v in w.items()}
    m = dict(heads=H, dim=d, vdim=vd, tau=tau)
    xs = [torch.randn(n, W, generator=g) for n in lengths]
    refs = [G.gated_linear_attention(x.double(), wd, "", m, eps) * scale for x in xs]
    stack = torch.cat([w[k] for k in ("q", "k", "v", "g", "a1")]).to(DEV)

    def run(cuts):
        state = torch.zeros(4, H, d, vd, device=DEV)
        state[0] = 7.0                                             # another sequence's state must not be touched
        at, rows = [0, 0], [[], []]
        for s in range(len(cuts[0])):
            live = [b for b in range(2) if cuts[b][s] > 0]
            ns = [cuts[b][s] for b in live]
            step = _step(ns, [slots[b] for b in live])
            x = torch.cat([xs[b][at[b]:at[b] + n] for b, n in zip(live, ns)]).to(DEV)
            out = torch.empty(x.shape[0], H * vd, device=DEV)
            K.gla(x @ stack.T, state, w["a2"].to(DEV), w["a2.b"].to(DEV), w["norm"].to(DEV), out, step, H, d, vd, rank, tau,
                  eps, scale)
            o = 0
            for b, n in zip(live, ns):
                rows[b].append(out[o:o + n].cpu())
                o += n
                at[b] += n
        assert float((state[0] - 7.0).abs().max()) == 0.0
        return [torch.cat(r) for r in rows]

    # whole (chunks of 64 with a ragged last one), portions that start chunks elsewhere, short portions, token by token
    for cuts in ([[150], [37]], [[64, 86], [0, 37]], [[2, 33, 114, 1], [1, 1, 33, 2]], [[1] * 150, [1] * 37 + [0] * 113],
                 [[100, 16, 34], [5, 32, 0]]):
        got = run(cuts)
        for b in range(2):
            assert worst(got[b], refs[b]) <= 2e-5, (cuts, b)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (6, 3, 1, 1), (9, 3, 3, 1), (4, 1, 2, 1), (4, 2, 4, 2), (64, 6, 8, 3), (40, 8, 1, 1)])
def test_router_choice_and_experts(E, top, groups, keep):
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(E + top)
    T, W, F, limit = 77, 24, 12, 0.7
    x = torch.randn(T, W, generator=g)
    w = {"router": torch.randn(E, W, generator=g) * 0.5, "correction": torch.randn(E, generator=g) * 0.6}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = torch.randn(F, W, generator=g) * 0.4, torch.randn(F, W, generator=g) * 0.4
        w[f"e{e}.down"] = torch.randn(W, F, generator=g) * 0.4
    wd = {k: v.double() for k, v in w.items()}
    r = dict(experts=E, top=top)
    if groups > 1:
        r["groups"] = dict(count=groups, keep=keep)
    idx, wt = G.route(x.double(), wd, "", r)
    z = (x @ w["router"].T).to(DEV)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    K.moe_select(z, w["correction"].to(DEV), ids, wts, top, groups, keep)
    assert torch.equal(ids.cpu().long().sort(dim=1).values, idx.sort(dim=1).values)
    order, ref_order = ids.cpu().long().argsort(dim=1), idx.argsort(dim=1)
    assert worst(wts.cpu().gather(1, order), wt.gather(1, ref_order)) <= 1e-5
    ref = G.moe_ff(x.double(), wd, "", dict(router=r, expert=dict(limit=limit)))
    gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(DEV)
    dn = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(DEV)
    y = torch.full((T, W), 0.25, device=DEV)
    K.moe_experts(x.to(DEV), ids, wts, gu, dn, y, top, limit)
    assert worst(y - 0.25, ref) <= 1e-5
    # one token alone gives the same row as in the batch, bit for bit
    y1 = torch.zeros(1, W, device=DEV)
    K.moe_experts(x[5:6].to(DEV), ids[5:6].contiguous(), wts[5:6].contiguous(), gu, dn, y1, top, limit)
    y0 = torch.zeros(T, W, device=DEV)
    K.moe_experts(x.to(DEV), ids, wts, gu, dn, y0, top, limit)
    assert torch.equal(y1[0], y0[5])


@pytest.mark.parametrize("T,W,F,E,top", [(150, 72, 40, 8, 2), (3, 64, 136, 16, 4), (700, 200, 64, 4, 3)])
def test_experts_on_the_tensor_cores(T, W, F, E, top):
    """bfloat16 rows and weights whose sizes are multiples of eight take the tensor-core tiles: the result is the
    plain one on the same rounded operands, up to the rounding of the activation; a token's row does not depend on
    the batch it is in."""
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(T + W)
    limit = 1.3
    x = torch.randn(T, W, generator=g).bfloat16()
    w = {"router": torch.randn(E, W, generator=g) * 0.5, "correction": torch.zeros(E)}
    for e in range(E):
        for n, shape in (("gate", (F, W)), ("up", (F, W)), ("down", (W, F))):
            w[f"e{e}.{n}"] = (torch.randn(shape, generator=g) * 0.3).bfloat16()
    wd = {k: v.double() for k, v in w.items()}
    r = dict(experts=E, top=top)
    idx, wt = G.route(x.double(), wd, "", r)
    ref = G.moe_ff(x.double(), wd, "", dict(router=r, expert=dict(limit=limit)))
    gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(DEV)
    dn = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(DEV)
    ids, wts = idx.int().to(DEV).contiguous(), wt.float().to(DEV).contiguous()
    y = torch.zeros(T, W, device=DEV)
    K.moe_experts(x.to(DEV), ids, wts, gu, dn, y, top, limit)
    assert worst(y, ref) <= 8e-3
    t = T // 2
    y1 = torch.zeros(1, W, device=DEV)
    K.moe_experts(x[t:t + 1].to(DEV), ids[t:t + 1].contiguous(), wts[t:t + 1].contiguous(), gu, dn, y1, top, limit)
    assert torch.equal(y1[0], y[t])


@pytest.mark.parametrize("T,W,F,E,top,blk", [(400, 128, 64, 4, 2, 64), (700, 256, 384, 8, 3, 128), (300, 128, 192, 16, 4, 64)])
def test_experts_as_grouped_products_of_the_tile_kernel(T, W, F, E, top, blk):
    """Many pairs, gate and up rows in blocks: rows gathered into 128-row tiles of one expert each, two grouped
    products of the tcgen05 tile kernel, the weighted sum by a scatter map. The same weights with few pairs take the
    mma.sync tiles (a decode step); both agree with the plain implementation."""
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(T + F)
    limit = 0.9
    x = torch.randn(T, W, generator=g).bfloat16()
    w = {"router": torch.randn(E, W, generator=g) * 0.5, "correction": torch.zeros(E)}
    for e in range(E):
        for n, shape in (("gate", (F, W)), ("up", (F, W)), ("down", (W, F))):
            w[f"e{e}.{n}"] = (torch.randn(shape, generator=g) * 0.3).bfloat16()
    w["correction"][E - 1] = -10.0                              # an expert nobody chooses: its tiles are passed over
    wd = {k: v.double() for k, v in w.items()}
    r = dict(experts=E, top=top)
    idx, wt = G.route(x.double(), wd, "", r)
    assert E - 1 not in idx
    ref = G.moe_ff(x.double(), wd, "", dict(router=r, expert=dict(limit=limit)))
    gu = torch.stack([torch.stack([w[f"e{e}.gate"].reshape(F // blk, blk, W), w[f"e{e}.up"].reshape(F // blk, blk, W)], dim=1)
                      .reshape(2 * F, W) for e in range(E)]).to(DEV).contiguous()
    dn = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(DEV)
    ids, wts = idx.int().to(DEV).contiguous(), wt.float().to(DEV).contiguous()
    y = torch.full((T, W), 0.5, device=DEV)
    K.moe_experts(x.to(DEV), ids, wts, gu, dn, y, top, limit, glu_block=blk)
    torch.cuda.synchronize()
    K.check_status(torch.device(DEV))
    assert worst(y - 0.5, ref) <= 8e-3
    few = slice(T // 2, T // 2 + 5)
    y5 = torch.zeros(5, W, device=DEV)
    K.moe_experts(x[few].to(DEV), ids[few].contiguous(), wts[few].contiguous(), gu, dn, y5, top, limit, glu_block=blk)
    assert worst(y5, ref[few]) <= 8e-3
    assert worst(y5, (y - 0.5)[few].cpu()) <= 8e-3


def test_activations_and_attention_with_values_of_another_size():
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(3)
    z = 3 * torch.randn(19, 70, generator=g)
    out = torch.empty(19, 70, device=DEV)
    K.gelu_tanh(z.to(DEV), out)
    assert worst(out, G.gelu_tanh(z.double())) <= 1e-6
    gu = 2 * torch.randn(19, 2 * 35, generator=g)
    out = torch.empty(19, 35, device=DEV)
    K.clamped_glu(gu.to(DEV), out, 1.1)
    gg, uu = gu[:, :35].double().clamp(max=1.1), gu[:, 35:].double().clamp(-1.1, 1.1)
    assert worst(out, gg * torch.sigmoid(1.702 * gg) * (uu + 1)) <= 1e-6
    # generic attention: keys of 12, values of 20, a window of 9, two heads on one kv head
    T, nh, d, vd, win = 50, 2, 12, 20, 9
    q, k, v = torch.randn(T, nh, d, generator=g), torch.randn(T, 1, d, generator=g), torch.randn(T, 1, vd, generator=g)
    kpool, vpool = torch.zeros(3, 1, 64, d, device=DEV), torch.zeros(3, 1, 64, vd, device=DEV)
    kpool[2, 0, :T], vpool[2, 0, :T] = k[:, 0].to(DEV), v[:, 0].to(DEV)
    step = _step([T])
    meta = SimpleNamespace(token_seq=step.token_seq, positions=step.positions, page_size=64,
                           seq_slot=torch.zeros(1, dtype=torch.int32, device=DEV),
                           page_table=torch.tensor([[2]], dtype=torch.int32, device=DEV))
    out = torch.empty(T, nh * vd, device=DEV)
    K.attention_generic(q.reshape(T, -1).to(DEV), kpool, vpool, out, meta, nh, 1, d, win, 0.4, vd=vd)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    see = (j <= i) & (i - j < win)
    ref = torch.stack([torch.softmax(((q[:, h].double() @ k[:, 0].double().T) * 0.4).masked_fill(~see, -math.inf), -1)
                       @ v[:, 0].double() for h in range(nh)], dim=1)
    assert worst(out, ref.reshape(T, -1)) <= 1e-5


# ---------------------------------------------------------------------------------------------- whole models
LENGTHS = {"a": [1, 2, 23, 64, 65, 150], "b": [3, 63, 129, 140, 70, 9], "c": [5, 1, 40, 100, 66, 31],
           "d": [2, 70, 1, 33, 129, 64]}


def refs_of(m, reqs):
    ref = {}
    for rid, toks in reqs.items():
        logits = logits_of(m, toks)
        for p in range(len(toks)):
            ref[(rid, p)] = logits[p]
    return ref


# A router's choice is a step function of its input: where two experts' (or groups') scores lie closer than bfloat16
# rounding moves them, the bfloat16 run may choose the other one, and that token's logits (and, fading, those of the
# tokens that see it) differ by far more than rounding. The 32-bit runs must agree everywhere; the bfloat16 runs may
# leave this share of rows outside the tolerance.
CLOSE_CALLS = 0.08


def compare(got, ref, tol, what, allow=0.0):
    assert set(got) == set(ref), what
    scale = max(float(v.abs().max()) for v in ref.values())
    errs = sorted(((float((row.double() - ref[k].double()).abs().max()) / scale, k) for k, row in got.items()),
                  key=lambda x: x[0] if x[0] == x[0] else 9e9)
    assert all(e == e for e, _ in errs), what
    over = [x for x in errs if x[0] > tol]
    assert len(over) <= allow * len(errs), \
        f"{what}: {len(over)} of {len(errs)} rows beyond {tol:.1e}, the worst {over[-1][0]:.3e} of the largest logit at {over[-1][1]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_every_cut_agrees_with_plain(models, name, dtype, tmp_path):
    m = models[name]
    reqs = {f"r{i}": tiny.random_prompt(m.vocab, n, 31 * i + n) for i, n in enumerate(LENGTHS[name])}
    ref = refs_of(m, reqs)
    decode = {rid: d for rid, d in zip(reqs, [0, 1, 22, 40, 3, 90])}
    cuts = {"whole": traces.whole(reqs), "tail": traces.tail_one_by_one(reqs, 45),
            "ragged": traces.ragged_batches(reqs, 3, decode),
            "ragged_pairs": traces.ragged_batches(dict(reversed(list(reqs.items()))), 2, decode)}
    tol = {"float32": 2e-5, "bfloat16": 3e-2}[dtype]
    allow = 0.0 if dtype == "float32" else CLOSE_CALLS
    results = {}
    for cut, steps in cuts.items():
        out = tmp_path / cut
        traces.run_in_process(m.folder, dtype, steps, str(out))          # a cache that holds just this trace: slots and pages come back
        results[cut] = traces.collect(steps, str(out), m.vocab)
        compare(results[cut], ref, tol, f"{name}/{dtype}/{cut}", allow)
    for cut in ("tail", "ragged", "ragged_pairs"):
        compare(results[cut], results["whole"], tol, f"{name}/{dtype}: {cut} against whole", allow)


def test_a_long_prompt_takes_the_grouped_expert_products_and_decoding_the_small_tiles(tmp_path):
    """A width and expert size that the tcgen05 tile kernel takes: a prompt of 300 tokens (600 pairs) runs its experts
    as grouped products, the decode steps behind it on the mma.sync tiles, the 32-bit mode on FFMA tiles; all agree with
    the plain implementation."""
    from spissa_b200.csrc import lib as K
    cfg = model(128, 180, [par(left(4, 2, 32, 32, conv=3, rot=16, window=100), 2, 16, 32, 8.0, 0.8, 0.6),
                           par(left(2, 2, 64, 64, conv=2, rot=64, window=40), 1, 32, 64, 4.0, 1.0, 1.0)],
                [moe(8, 2, 64, 2.0, groups=(2, 1), shared=(64, 2.0)), moe(4, 3, 128, 1.0)], streams=2)
    pcfg, w = make(cfg, tmp_path, seed=41, std=0.07, norm_std=0.1)
    m = SimpleNamespace(cfg=pcfg, w=w)
    toks = tiny.random_prompt(180, 330, 8)
    ref = logits_of(m, toks)
    for dtype, tol, allow in (("float32", 2e-5, 0.0), ("bfloat16", 3e-2, CLOSE_CALLS)):
        eng = Engine.from_folder(str(tmp_path), dtype=dtype, max_tokens=64 * 7, max_seqs=1)
        before = K.launches
        s = eng.acquire()
        rows = [eng.step([(s, toks[:300], list(range(300)))]).cpu()]
        rows += [eng.step([(s, [t], [0])]).cpu() for t in toks[300:]]
        eng.release(s)
        got = {("p", i): r for i, r in enumerate(torch.cat(rows))}
        compare(got, {("p", i): r for i, r in enumerate(ref)}, tol, dtype, allow)
        if dtype == "bfloat16":
            layer = eng.model.layers[0].ffn
            assert layer.glu_block == 64 and eng.model.layers[1].ffn.glu_block == 128
    assert "tc_gemm" in K.loaded_libraries()


@pytest.mark.parametrize("name", ["a", "d"])
def test_portions_of_a_prompt_down_to_two_tokens(models, name):
    m = models[name]
    toks = tiny.random_prompt(m.vocab, 150, 77)
    ref = logits_of(m, toks)
    other = tiny.random_prompt(m.vocab, 80, 78)
    ref_other = logits_of(m, other)
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 6, max_seqs=3)
    for sizes in ([2, 2, 3, 57, 1, 64, 21], [64, 64, 22], [1, 1, 2, 146]):
        s, s2 = engine.acquire(), engine.acquire()
        at, rows, rows2 = 0, [], []
        for n in sizes:
            entries = [(s, toks[at:at + n], list(range(n)))]
            lo2, hi2 = min(at, 80), min(at + n, 80)                      # the second request's portions end earlier
            if hi2 > lo2:
                entries.append((s2, other[lo2:hi2], list(range(hi2 - lo2))))
            got = engine.step(entries).cpu()
            rows.append(got[:n])
            rows2.append(got[n:])
            at += n
        assert worst(torch.cat(rows), ref) <= 2e-5, sizes
        assert worst(torch.cat(rows2), ref_other) <= 2e-5, sizes
        engine.release(s)
        engine.release(s2)
    engine.cache.check()
    assert engine.cache.slots.held_count == 0


def test_slots_and_pages_that_are_used_again_start_clean(models):
    m = models["a"]
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 3, max_seqs=2)
    for round_ in range(3):
        reqs = [tiny.random_prompt(m.vocab, n, 5 * round_ + n) for n in ((100, 30), (7, 120), (64, 65))[round_]]
        slots = [engine.acquire() for _ in reqs]
        got = engine.step([(s, r[:-2], [len(r) - 3]) for s, r in zip(slots, reqs)]).cpu()
        for b, r in enumerate(reqs):
            assert worst(got[b], logits_of(m, r[:-2])[-1]) <= 2e-5
        for i in (2, 1):
            got = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
        for b, r in enumerate(reqs):
            assert worst(got[b], logits_of(m, r)[-1]) <= 2e-5
        for s in slots:
            engine.release(s)
        engine.cache.check()


def test_long_decoding_lets_windows_pass_over_decoded_tokens_and_returns_pages(models):
    m = models["a"]                              # windows of 20, 7 and 70
    toks = tiny.random_prompt(m.vocab, 230, 3)
    ref = logits_of(m, toks)
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 3e-2)):
        engine = Engine.from_folder(m.folder, dtype=dtype, max_tokens=64 * 4, max_seqs=1)
        s = engine.acquire()
        engine.step([(s, toks[:10], [])])
        rows = torch.cat([engine.step([(s, [t], [0])]).cpu() for t in toks[10:]])
        got = {("long", i): r for i, r in enumerate(rows)}
        compare(got, {("long", i): r for i, r in enumerate(ref[10:])}, tol, dtype, 0.0 if dtype == "float32" else CLOSE_CALLS)
        for g in engine.cache.kv_groups.values():                       # the windowed groups gave their first pages back
            flags = [p is not None for p in engine.cache.seqs[s].pages[g.name]]
            assert flags[-1] and not flags[0]
        engine.release(s)
        engine.cache.check()


# ---------------------------------------------------------------------------------------------- one key that matters
NEEDLE, DIRECTION, CONST = 7, 0, 1


def needle_model(window, dim=16, rot=8):
    """One layer whose attention gives almost all its weight to the key of token ``NEEDLE`` wherever that key is
    visible, and whose values make the needle's presence large in the logits. The convolutions pass the current token
    only, so that the needle's key stands at the needle's position alone."""
    cfg = model(32, 64, [par(left(2, 1, dim, 16, conv=3, rot=rot, window=window, scale=1.0), 1, 4, 4, 8.0, 1.0, 0.05)], [None],
                streams=2)

    def patch(w):
        w["embed"][:, DIRECTION] = 0.0
        w["embed"][NEEDLE, DIRECTION] = 6.0
        w["embed"][:, CONST] = 5.0                                # after the norm every token has the same large entry here
        w["l0.norm1"][DIRECTION] = 1.0
        w["l0.norm1"][CONST] = 1.0
        w["l0.hc1.in"][:] = 0.5
        for n in ("q", "k", "v"):
            w[f"l0.mix.left.{n}.conv"].zero_()
            w[f"l0.mix.left.{n}.conv"][:, -1] = 1.0
            w[f"l0.mix.left.{n}"][:, DIRECTION] = 0.0
            w[f"l0.mix.left.{n}"][:, CONST] = 0.0
        j = dim - 1                                               # a dim that is not rotated
        w["l0.mix.left.k"][j, :] = 0.0
        w["l0.mix.left.k"][j, DIRECTION] = 4.0                    # the needle's key points along dim j, nobody else's does
        for h in range(2):
            w["l0.mix.left.q"][h * dim + j, CONST] = 4.0          # every query looks along dim j
        w["l0.mix.left.v"][:, DIRECTION] = 3.0                    # and the needle's value stands out

    return cfg, patch


@pytest.mark.parametrize("window", [20, 64, 70, 130])
def test_a_key_just_inside_and_just_outside_the_window(tmp_path, window):
    cfg, patch = needle_model(window)
    pcfg, w = make(cfg, tmp_path, seed=21, std=0.05, norm_std=0.0, patch=patch)
    m = SimpleNamespace(cfg=pcfg, w=w)
    T = 200
    base = [t if t != NEEDLE else NEEDLE + 1 for t in tiny.random_prompt(64, T, 99)]
    places = [T - 1 - (window - 1), T - 1 - window, T - 2 - (window - 1), 63, 64, T - 1]
    engines = {dt: Engine.from_folder(str(tmp_path), dtype=dt, max_tokens=64 * 4, max_seqs=1) for dt in ("float32", "bfloat16")}
    last = {}
    for place in places:
        toks = list(base)
        toks[place] = NEEDLE
        ref = logits_of(m, toks)
        last[place] = ref[-1]
        for dt, tol in (("float32", 2e-5), ("bfloat16", 3e-2)):
            eng = engines[dt]
            s = eng.acquire()
            got = eng.step([(s, toks, [T - 2, T - 1])]).cpu()                   # in a prompt
            assert worst(got, ref[-2:]) <= tol, (place, dt, "prompt")
            eng.release(s)
            s = eng.acquire()
            eng.step([(s, toks[:T - 40], [])])
            for t in toks[T - 40:T - 2]:
                eng.step([(s, [t], [])])
            got = torch.cat([eng.step([(s, [t], [0])]) for t in toks[T - 2:]]).cpu()   # decoded, pages returned meanwhile
            assert worst(got, ref[-2:]) <= tol, (place, dt, "decoded")
            eng.release(s)
    # the test can see the edge: a needle inside changes the last logits by far more than the tolerance
    inside, outside = last[T - 1 - (window - 1)], last[T - 1 - window]
    assert float((inside - outside).abs().max() / inside.abs().max()) > 0.2


def test_a_far_key_among_hundreds_without_a_window(tmp_path):
    cfg, patch = needle_model(None)
    pcfg, w = make(cfg, tmp_path, seed=22, std=0.05, norm_std=0.0, patch=patch)
    m = SimpleNamespace(cfg=pcfg, w=w)
    T = 700
    base = [t if t != NEEDLE else NEEDLE + 1 for t in tiny.random_prompt(64, T, 5)]
    plain_last = logits_of(m, base)[-1]
    eng = Engine.from_folder(str(tmp_path), dtype="float32", max_tokens=64 * 11, max_seqs=1)
    for place in (1, 64, 383, 640):
        toks = list(base)
        toks[place] = NEEDLE
        ref = logits_of(m, toks)
        assert float((ref[-1] - plain_last).abs().max() / ref[-1].abs().max()) > 0.2
        s = eng.acquire()
        head = eng.step([(s, toks[:-1], [T - 2])]).cpu()
        tail = eng.step([(s, [toks[-1]], [0])]).cpu()
        eng.release(s)
        assert worst(head[0], ref[-2]) <= 2e-5 and worst(tail[0], ref[-1]) <= 2e-5, place


def test_the_first_tokens_of_a_sequence_see_zeros_before_its_start(models):
    """Tokens 0 … taps−2 convolve over places before the sequence: a slot whose last sequence left values there must
    not leak them, neither in a prompt nor when the first tokens come one by one."""
    m = models["a"]
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 2, max_seqs=1)
    for toks in (tiny.random_prompt(m.vocab, 40, 1), tiny.random_prompt(m.vocab, 6, 2)):
        ref = logits_of(m, toks)
        s = engine.acquire()
        assert worst(engine.step([(s, toks, list(range(len(toks))))]).cpu(), ref) <= 2e-5
        engine.release(s)
        s = engine.acquire()
        rows = [engine.step([(s, [t], [0])]).cpu() for t in toks[:6]]
        assert worst(torch.cat(rows), ref[:6]) <= 2e-5
        engine.release(s)


# ---------------------------------------------------------------------------------------------- generation, the program
def greedy_plain(m, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(logits_of(m, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("name", ["a", "c"])
def test_greedy_generation_through_the_entry_point(models, name):
    m = models[name]
    prompts = [tiny.random_prompt(m.vocab, n, 7 * n) for n in (1, 9, 70, 30)]
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 8, max_seqs=3)     # two batches
    results, metrics = engine.generate(prompts, 12, SamplingParams(), stop_ids=[])
    for p, r in zip(prompts, results):
        ids = list(p)
        for tok in r.tokens:                                   # along the engine's own tokens: the chosen one is the largest
            row = logits_of(m, ids)[-1]
            assert float(row.max() - row[tok]) <= 2e-5 * float(row.abs().max()), f"prompt of {len(p)}"
            ids.append(tok)
        assert len(r.tokens) == 12 and r.finish_reason == "length"
    assert metrics.generated_tokens == 12 * len(prompts)
    engine.cache.check()
    assert engine.cache.slots.held_count == 0
    # bfloat16 and sampling run through the same loop
    engine = Engine.from_folder(m.folder, dtype="bfloat16", max_tokens=64 * 8)
    results, _ = engine.generate(prompts, 6, SamplingParams(temperature=0.8, top_k=20, seed=3), stop_ids=[])
    assert all(len(r.tokens) == 6 and all(0 <= t < m.vocab for t in r.tokens) for r in results)


def test_trace_program_on_a_model_of_this_design(models, tmp_path):
    m = models["b"]
    reqs = {f"q{i}": tiny.random_prompt(m.vocab, n, n) for i, n in enumerate([40, 3, 90])}
    steps = traces.ragged_batches(reqs, 3, {"q0": 5, "q1": 2, "q2": 30})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", m.folder, "--dtype", "bfloat16",
         "--out", str(out), "--max-tokens", str(traces.tokens_needed(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    compare(traces.collect(steps, str(out), m.vocab), refs_of(m, reqs), 3e-2, "trace program", CLOSE_CALLS)


def test_command_line_generates_from_a_folder_and_from_a_configuration_with_random_weights(models, tmp_path):
    m = models["c"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "bin", "spissa-b200")
    prompt = tiny.random_prompt(m.vocab, 12, 4)
    proc = subprocess.run([sys.executable, exe, "generate", m.folder, "--token-ids", ",".join(map(str, prompt)),
                           "--max-new-tokens", "5", "--dtype", "fp32", "--ctx", "128"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[0])
    assert line["tokens"] == greedy_plain(m, prompt, 5) and line["finish_reason"] == "length"
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["a"]))
    proc = subprocess.run([sys.executable, exe, "generate", "--random", str(cfg_file), "--token-ids", "1,2,3",
                           "--token-ids", "9,8,7,6,5", "--max-new-tokens", "4", "--temp", "0.7", "--seed", "2", "--ctx", "128"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(x) for x in proc.stdout.strip().splitlines()]
    assert [len(x["tokens"]) for x in lines] == [4, 4]
