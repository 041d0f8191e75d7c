"""The Duzinex parts and the whole decoder against the plain implementation in ``plain/duzinex_plain.py``.

Each mechanism alone (kernel against its formula), then small models with random weights under every way of cutting
the work: whole prompts, token-by-token decoding, portions down to two tokens, batches of unequal requests, slots
and pages used again, long decoding with a window that passes over decoded tokens, greedy generation through
``Engine.generate``, and the trace program. Where random weights would hide a fault (one key among many, the
window's and the kept tokens' edges), the weights are made so that one key dominates a map.
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
from plain import duzinex_plain as D
from spissa_b200 import Engine, SamplingParams
from spissa_b200.config import config_from_dict
from spissa_b200.weights import write_random_model, write_safetensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def att(heads, kv, dim, vdim, window=None, keep=0, rot=None, base=10000.0, cap=None, diff=0.3, scale=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, diff=diff, scale=scale or 1.0 / math.sqrt(dim), softcap=cap)
    if window:
        m["mask"] = dict(size=window, keep_first=keep)
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    return dict(type="attention", mixer=m)


def ret(heads, dim, vdim, decay):
    return dict(type="retention", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay))


def gru(width):
    return dict(type="mingru", mixer=dict(width=width))


def model(width, vocab, layers, ffs, loop=None, scale=3.0, eps=1e-5):
    out = dict(architecture="Duzinex", vocab=vocab, width=width, embedding=dict(scale=scale), norm=dict(eps=eps),
               layers=[dict(l, mlp=(dict(kind="dense", ff=f) if f else None)) for l, f in zip(layers, ffs)])
    if loop:
        out["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return out


# sizes that differ from one another everywhere: grouped, multi-head and single-head attention; rotation over a part
# of the dims or all; windows below and above a page; kept tokens none, a few, more than a page; value sizes other than
# twice the map size; retention with dim != vdim; a recurrent width other than the feed-forward's; layers without a
# feed-forward; loops of 1, 2 and 3 passes, over a part or all of the layers, or none
CONFIGS = {
    "a": model(64, 200, [att(4, 2, 16, 32, window=20, keep=3, rot=8, cap=5.0), gru(96), ret(3, 8, 16, [0.9, 0.97, 0.5]),
                         att(2, 1, 8, 32, window=7, keep=0, rot=8, base=100.0, diff=0.7)],
               [80, None, 48, 72], loop=(1, 3, 3)),
    "b": model(96, 333, [ret(1, 16, 40, [0.99]), att(3, 3, 12, 20, window=70, keep=66, rot=4, cap=None, diff=0.1),
                         gru(40)], [56, 120, None], loop=None, scale=1.0, eps=1e-3),
    "c": model(48, 150, [gru(48), att(1, 1, 32, 16, window=None, rot=32, base=500.0, cap=2.0, diff=0.5),
                         ret(2, 24, 8, [0.8, 0.999])], [96, 64, 32], loop=(0, 3, 2), scale=7.5),
    # nothing a multiple of four: the paths without wide loads, an odd map size of which four dims turn
    "d": model(50, 97, [att(2, 1, 7, 9, window=9, keep=2, rot=4, cap=3.0, diff=0.4), ret(2, 5, 7, [0.7, 0.95]), gru(22)],
               [30, 26, 34], loop=(0, 2, 2), scale=2.0),
}
INIT = {"a": dict(seed=5, std=0.08, norm_std=0.2), "b": dict(seed=9, std=0.06, norm_std=0.1),
        "c": dict(seed=13, std=0.1, norm_std=0.3), "d": dict(seed=17, std=0.12, norm_std=0.2)}


def make(cfg, folder, seed, std, norm_std, patch=None):
    write_random_model(config_from_dict(cfg), folder, seed=seed, std=std, norm_std=norm_std)
    pcfg, w = D.read_model_folder(folder)
    # the random-weights mode gives every shift a small value and every alpha and activation number one value:
    # spread them, so that a shift taken from the wrong token or a swapped coefficient shows
    g = torch.Generator().manual_seed(seed)
    for name in sorted(w):
        if name.endswith(".shift"):
            w[name] = torch.rand(w[name].shape, generator=g).to(w[name].dtype)
        elif name.endswith(".alpha"):
            w[name] = (0.2 + 0.6 * torch.rand((), generator=g)).to(w[name].dtype)
        elif name.endswith(".act"):
            w[name] = torch.tensor([0.9, -0.4, 0.25, 0.1]).to(w[name].dtype) * (0.5 + torch.rand(4, generator=g)).to(w[name].dtype)
        elif name.split(".")[-1] in ("lq1", "lk1", "lq2", "lk2"):
            w[name] = (0.5 * torch.randn(w[name].shape, generator=g)).to(w[name].dtype)
    if patch:
        patch(w)
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    return D.read_model_folder(folder)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"dz_{name}")
        pcfg, w = make(cfg, folder, **INIT[name])
        out[name] = SimpleNamespace(folder=str(folder), cfg=pcfg, w=w, vocab=cfg["vocab"])
    return out


def worst(got, ref):
    return float((got.double().cpu() - ref.double()).abs().max() / ref.abs().max())


# ---------------------------------------------------------------------------------------------- each mechanism alone
def _step(lengths, slots=None):
    """The device arrays a kernel wants of a step with sequences of these lengths."""
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    seq = [b for b, n in enumerate(lengths) for _ in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(seq_start=i32(starts), seq_slot=i32(slots or list(range(len(lengths)))), token_seq=i32(seq),
                           n_seqs=len(lengths), all_single=all(n == 1 for n in lengths), max_new=max(lengths),
                           host=dict(new_counts=list(lengths)))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_and_polynorm_kernels(out_dtype):
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(1)
    x = 3 * torch.randn(37, 200, generator=g)
    w = {"n": torch.randn(200, generator=g), "n.b": torch.randn(200, generator=g), "n.alpha": torch.tensor(0.37)}
    out = torch.empty(37, 200, dtype=out_dtype, device=DEV)
    K.dyt_norm(x.to(DEV), w["n"].to(DEV), w["n.b"].to(DEV), w["n.alpha"].reshape(1).to(DEV), out)
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    assert worst(out, D.dynamic_tanh(x.double(), {k: v.double() for k, v in w.items()}, "n")) <= tol
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=DEV)
    some = torch.empty(3, 200, dtype=out_dtype, device=DEV)
    K.dyt_norm(x.to(DEV), w["n"].to(DEV), w["n.b"].to(DEV), w["n.alpha"].reshape(1).to(DEV), some, rows)
    assert torch.equal(some, out[rows.long()])
    # PolyNorm: rows of a size that no block divides, coefficients all different, one large entry in a row
    z = torch.randn(19, 333, generator=g)
    z[3, 17] = 40.0
    coef = torch.tensor([0.7, -1.3, 0.45, 0.2])
    act = torch.empty(19, 333, dtype=out_dtype, device=DEV)
    K.polynorm(z.to(DEV), coef.to(DEV), act, 1e-4)
    zz = z.double()
    ref = 0.7 * D.unit_rms(zz, 1e-4) - 1.3 * D.unit_rms(zz ** 2, 1e-4) + 0.45 * D.unit_rms(zz ** 3, 1e-4) + 0.2
    assert worst(act, ref) <= (5e-6 if out_dtype == torch.float32 else 5e-3)
    # a bias on the rows of a 32-bit matrix
    rows32 = x.clone().to(DEV)
    bias = torch.randn(200, generator=g).to(out_dtype)
    K.add_bias(rows32, bias.to(DEV))
    assert worst(rows32, x.double() + bias.double()) <= 1e-6


def test_token_shift_kernel_carries_the_last_row_in_the_state():
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(2)
    H = 72
    a = torch.randn(30, H, generator=g)
    mu = torch.rand(H, generator=g)
    lengths = [11, 1, 18]
    ref = torch.cat([D.token_shift(s.double(), mu.double()) for s in a.split(lengths)])
    state = torch.zeros(5, H, device=DEV)
    # whole, on slots 3, 0, 4
    out = torch.empty(30, H, device=DEV)
    K.token_shift(a.to(DEV), mu.to(DEV), state, out, _step(lengths, [3, 0, 4]))
    assert worst(out, ref) <= 1e-6
    assert torch.equal(state[[3, 0, 4]].cpu(), a[[10, 11, 29]]) and float(state[[1, 2]].abs().sum()) == 0
    # the same cut in two: the second part's first tokens read what the first part left
    state.zero_()
    first, second = [4, 1, 16], [7, 0, 2]
    parts = a.split(lengths)
    head = torch.cat([p[:n] for p, n in zip(parts, first)])
    tail = torch.cat([p[n:] for p, n in zip(parts, first)])
    o1 = torch.empty(head.shape[0], H, device=DEV)
    K.token_shift(head.to(DEV), mu.to(DEV), state, o1, _step(first, [3, 0, 4]))
    o2 = torch.empty(tail.shape[0], H, device=DEV)
    K.token_shift(tail.to(DEV), mu.to(DEV), state, o2, _step([7, 2], [3, 4]))
    got = torch.cat([o1[:4], o2[:7], o1[4:5], o1[5:], o2[7:]])
    assert worst(got, ref) <= 1e-6
    # one token each (the state is stored by the same launch)
    for t in range(2):
        o = torch.empty(2, H, device=DEV)
        K.token_shift(a[[5 + t, 20 + t]].to(DEV), mu.to(DEV), state, o, _step([1, 1], [1, 2]))
    assert worst(o[0], (a[6] + (a[5] - a[6]) * mu)) <= 1e-6 and torch.equal(state[2].cpu(), a[21])


@pytest.mark.parametrize("heads,dim,vdim", [(3, 8, 16), (1, 40, 24), (2, 16, 70), (2, 128, 130), (1, 72, 256), (1, 130, 8),
                                             (2, 100, 40), (2, 32, 32)])
def test_retention_kernel(heads, dim, vdim):
    """Sequences of 50 and 39 tokens run in chunks (where the key size allows), the single token and the portions
    below token by token; a chunk boundary lies inside nothing here, the next test crosses several."""
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(3)
    T, lengths = 90, [50, 1, 39]
    W = 2 * heads * dim + 2 * heads * vdim
    proj = torch.randn(T, W, generator=g)
    decay = [0.5 + 0.499 * i / max(1, heads - 1) for i in range(heads)]
    # the formula with identity projections: a = proj, weights pick the columns
    eye = torch.eye(W, dtype=torch.float64)
    cut = [0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim, W]
    w = {"q": eye[cut[0]:cut[1]], "k": eye[cut[1]:cut[2]], "v": eye[cut[2]:cut[3]], "g": eye[cut[3]:cut[4]],
         "o": torch.eye(heads * vdim, dtype=torch.float64)}
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=decay)
    ref = torch.cat([D.retention(s.double(), w, "", m, 1e-5) for s in proj.split(lengths)])
    state = torch.zeros(4, heads, dim, vdim, device=DEV)
    out = torch.empty(T, heads * vdim, device=DEV)
    dec = torch.tensor(decay, device=DEV)
    K.retention(proj.to(DEV), state, dec, out, _step(lengths, [2, 0, 3]), heads, dim, vdim, 1e-5)
    assert worst(out, ref) <= 5e-6
    # in portions of 2, 1 and the rest: the state carries over
    state2 = torch.zeros_like(state)
    seqs = proj.split(lengths)
    a, b = seqs[0], seqs[2]
    outs = {0: [], 2: []}
    for lo, hi in ((0, 2), (2, 3), (3, 39)):
        part = torch.cat([a[lo:hi], b[lo:hi]])
        o = torch.empty(part.shape[0], heads * vdim, device=DEV)
        K.retention(part.to(DEV), state2, dec, o, _step([hi - lo, hi - lo], [2, 3]), heads, dim, vdim, 1e-5)
        outs[0].append(o[:hi - lo])
        outs[2].append(o[hi - lo:])
    assert worst(torch.cat(outs[0]), ref[:39]) <= 5e-6 and worst(torch.cat(outs[2]), ref[51:]) <= 5e-6


def test_recurrences_in_chunks_agree_with_token_by_token_across_chunk_borders():
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(8)
    heads, dim, vdim, W = 2, 32, 48, 70
    lengths = [200, 64, 65, 31]                      # 4 + 1 + 2 chunks, and one sequence below the chunked path's limit
    T = sum(lengths)
    proj = torch.randn(T, 2 * heads * dim + 2 * heads * vdim, generator=g).to(DEV)
    dec = torch.tensor([0.9, 0.999], device=DEV)
    start = torch.randn(5, heads, dim, vdim, generator=g).to(DEV)          # states that earlier steps left
    one_by_one = _step(lengths, [4, 1, 0, 2])
    one_by_one.max_new = 1                                                  # forces the token-by-token kernels
    s1, s2 = start.clone(), start.clone()
    o1 = torch.empty(T, heads * vdim, device=DEV)
    o2 = torch.empty_like(o1)
    K.retention(proj, s1, dec, o1, one_by_one, heads, dim, vdim, 1e-5)
    K.retention(proj, s2, dec, o2, _step(lengths, [4, 1, 0, 2]), heads, dim, vdim, 1e-5)
    assert worst(o2, o1.cpu()) <= 5e-6 and worst(s2, s1.cpu()) <= 5e-6
    assert torch.equal(s2[3], start[3])                                     # a slot that is not in the step
    pg = (2 * torch.randn(T, 3 * W, generator=g)).to(DEV)
    zb, xb = torch.randn(W, generator=g).to(DEV), torch.randn(W, generator=g).to(DEV)
    g0 = torch.randn(5, W, generator=g).to(DEV)
    g1, g2 = g0.clone(), g0.clone()
    y1 = torch.empty(T, W, device=DEV)
    y2 = torch.empty_like(y1)
    K.mingru(pg, zb, xb, g1, y1, one_by_one, W)
    K.mingru(pg, zb, xb, g2, y2, _step(lengths, [4, 1, 0, 2]), W)
    assert worst(y2, y1.cpu()) <= 2e-6 and worst(g2, g1.cpu()) <= 2e-6


def test_mingru_kernel_both_branches_of_the_candidate():
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(4)
    W, lengths = 50, [33, 2, 1]
    proj = 2 * torch.randn(36, 3 * W, generator=g)
    proj[:, W:W + 5] = 0.0                      # u exactly at the border (with a zero bias there): the u >= 0 side
    zb, xb = torch.randn(W, generator=g), torch.randn(W, generator=g)
    xb[:5] = 0.0
    eye = torch.eye(3 * W, dtype=torch.float64)
    w = {"z": eye[:W], "x": eye[W:2 * W], "g": eye[2 * W:], "z.b": zb.double(), "x.b": xb.double(),
         "o": torch.eye(W, dtype=torch.float64)}
    ref = torch.cat([D.mingru(s.double(), w, "", dict(width=W)) for s in proj.split(lengths)])
    u = proj[:, W:2 * W] + xb
    assert bool((u > 0).any()) and bool((u < 0).any()) and bool((u == 0).any())
    state = torch.zeros(3, W, device=DEV)
    out = torch.empty(36, W, device=DEV)
    K.mingru(proj.to(DEV), zb.to(DEV), xb.to(DEV), state, out, _step(lengths), W)
    assert worst(out, ref) <= 2e-6


@pytest.mark.parametrize("d,vd,H,G", [(16, 16, 2, 2), (32, 64, 4, 1), (64, 128, 2, 1), (128, 32, 1, 1), (128, 128, 2, 2), (24, 40, 2, 1),
                                      (12, 20, 3, 3), (16, 20, 16, 4), (64, 64, 2, 1), (32, 32, 4, 2), (16, 128, 1, 1)])
@pytest.mark.parametrize("window,keep,cap", [(0, 0, 0.0), (50, 0, 4.0), (70, 66, 0.0), (130, 3, 2.0)])
def test_differential_attention_kernels_over_pages(d, vd, H, G, window, keep, cap):
    """The prompt kernel on the tensor cores (where its sizes are built) and the kernels for any sizes (one warp per
    (token, head) for many pairs; for few pairs the warps of a CTA sharing the keys, with wide loads where the sizes
    allow), in bfloat16 and in 32-bit, against the formula: two sequences in one step, one of which already has 90 keys in the cache, on pages
    handed out in a scattered order."""
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(d * 1000 + vd + window)
    new, before = [150, 77], [0, 90]
    total = [n + b for n, b in zip(new, before)]
    bf = lambda t: t.to(torch.bfloat16).float()
    qs = [bf(torch.randn(t, H, 2, d, generator=g)) for t in total]
    ks = [bf(torch.randn(t, G, 2, d, generator=g)) for t in total]
    vs = [bf(torch.randn(t, G, vd, generator=g)) for t in total]
    lam, eps, out_scale, scale = 0.37, 1e-5, 0.8, 1.7 / d ** 0.5
    refs = []
    for q, k, v, n in zip(qs, ks, vs, new):
        q, k, v = q.double(), k.double(), v.double()
        see = D.visible(q.shape[0], window or None, keep)
        heads = []
        for h in range(H):
            kvh = h // (H // G)
            maps = []
            for i in range(2):
                s = (q[:, h, i] @ k[:, kvh, i].T) * scale
                if cap:
                    s = cap * torch.tanh(s / cap)
                maps.append(torch.softmax(s.masked_fill(~see, float("-inf")), dim=-1) @ v[:, kvh])
            heads.append(D.unit_rms(maps[0] - lam * maps[1], eps) * out_scale)
        refs.append(torch.cat(heads, dim=-1)[-n:])
    ref = torch.cat(refs)
    n_pages = 8
    order = [5, 2, 7, 0, 3, 6, 1, 4]
    table = torch.tensor([order[:3], order[3:6]], dtype=torch.int32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    meta = SimpleNamespace(page_table=table, page_size=64, seq_slot=i32([0, 1]),
                           token_seq=i32([0] * new[0] + [1] * new[1]),
                           positions=i32(list(range(before[0], total[0])) + list(range(before[1], total[1]))))
    q_new = torch.cat([q[-n:] for q, n in zip(qs, new)]).reshape(sum(new), H * 2 * d)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)):
        kp = torch.zeros(n_pages, G, 64, 2 * d, dtype=dtype, device=DEV)
        vp = torch.zeros(n_pages, G, 64, vd, dtype=dtype, device=DEV)
        for b in range(2):
            for pos in range(total[b]):
                page = int(table[b, pos // 64])
                kp[page, :, pos % 64] = ks[b][pos].reshape(G, 2 * d).to(dtype)
                vp[page, :, pos % 64] = vs[b][pos].to(dtype)
        qd = q_new.to(dtype).to(DEV)
        out = torch.empty(sum(new), H * vd, dtype=dtype, device=DEV)
        K.diff_attention(qd, kp, vp, out, meta, H, G, d, vd, window, keep, scale, cap, lam, eps, out_scale)
        assert worst(out, ref) <= tol, ("any sizes", dtype)
        if dtype == torch.bfloat16 and K.diff_flash_supported(d, vd, H, G, 64):
            fast = torch.empty_like(out)
            K.diff_flash_prefill(qd, kp, vp, fast, meta, i32([0, new[0], sum(new)]), 2, K.query_tiles(new, 64), H, G, d, vd,
                                 window, keep, scale, cap, lam, eps, out_scale)
            assert worst(fast, ref) <= tol, "tensor cores"
    assert K.diff_flash_supported(d, vd, H, G, 64) == (d in (16, 32, 64, 128) and vd in (16, 32, 64, 128))


# ---------------------------------------------------------------------------------------------- whole models
LENGTHS = {"a": [1, 2, 23, 64, 65, 150], "b": [3, 63, 129, 140, 70, 9], "c": [5, 1, 40, 100, 66, 31],
           "d": [2, 70, 1, 33, 129, 64]}


def refs_of(m, reqs):
    ref = {}
    for rid, toks in reqs.items():
        logits = D.model_logits(m.cfg, m.w, toks)
        for p in range(len(toks)):
            ref[(rid, p)] = logits[p]
    return ref


def compare(got, ref, tol, what):
    assert set(got) == set(ref), what
    scale = max(float(v.abs().max()) for v in ref.values())
    bad = max(((float((row.double() - ref[k]).abs().max()) / scale, k) for k, row in got.items()), key=lambda x: x[0] if x[0] == x[0] else 9e9)
    assert bad[0] <= tol, f"{what}: error {bad[0]:.3e} of the largest logit at {bad[1]} (allowed {tol:.1e})"


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
    results = {}
    for cut, steps in cuts.items():
        out = tmp_path / cut
        traces.run_in_process(m.folder, dtype, steps, str(out))          # a cache that holds just this trace: slots and pages come back
        results[cut] = traces.collect(steps, str(out), m.vocab)
        compare(results[cut], ref, tol, f"{name}/{dtype}/{cut}")
    scale = max(float(v.abs().max()) for v in ref.values())
    for cut in ("tail", "ragged", "ragged_pairs"):
        for key, row in results[cut].items():
            assert float((row - results["whole"][key]).abs().max()) / scale <= tol, f"{name}/{dtype}: {cut} at {key}"


@pytest.mark.parametrize("name", ["a", "b"])
def test_portions_of_a_prompt_down_to_two_tokens(models, name):
    m = models[name]
    toks = tiny.random_prompt(m.vocab, 150, 77)
    ref = D.model_logits(m.cfg, m.w, toks)
    other = tiny.random_prompt(m.vocab, 80, 78)
    ref_other = D.model_logits(m.cfg, m.w, other)
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
            assert worst(got[b], D.model_logits(m.cfg, m.w, r[:-2])[-1]) <= 2e-5
        for i in (2, 1):
            got = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
        for b, r in enumerate(reqs):
            assert worst(got[b], D.model_logits(m.cfg, m.w, r)[-1]) <= 2e-5
        for s in slots:
            engine.release(s)
        engine.cache.check()


def test_long_decoding_lets_windows_pass_over_decoded_tokens_and_returns_pages(models):
    m = models["a"]                              # windows of 20 and 7, three kept tokens
    toks = tiny.random_prompt(m.vocab, 230, 3)
    ref = D.model_logits(m.cfg, m.w, toks)
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 3e-2)):
        engine = Engine.from_folder(m.folder, dtype=dtype, max_tokens=64 * 4, max_seqs=1)
        s = engine.acquire()
        engine.step([(s, toks[:10], [])])
        rows = [engine.step([(s, [t], [0])]).cpu() for t in toks[10:]]
        assert worst(torch.cat(rows), ref[10:]) <= tol, dtype
        # the windowed groups gave pages back, but never the page of the kept first tokens
        held = {g.name: [p is not None for p in engine.cache.seqs[s].pages[g.name]] for g in engine.cache.kv_groups.values()}
        for g in engine.cache.kv_groups.values():
            flags = held[g.name]
            assert flags[-1] and not all(flags)
            assert flags[0] == (g.request.keep_first > 0)
        engine.release(s)
        engine.cache.check()


# ---------------------------------------------------------------------------------------------- one key that matters
NEEDLE, DIRECTION = 7, 0


def needle_model(folder, window, keep, dim=16, rot=8):
    """One attention layer (two heads on one kv head) whose first map gives almost all its weight to the key of token
    ``NEEDLE`` wherever that key is visible, and whose values make the needle's presence large in the logits."""
    cfg = model(32, 64, [att(2, 1, dim, 16, window=window, keep=keep, rot=rot, cap=30.0, diff=0.2, scale=1.0)], [None], scale=1.0)

    def patch(w):
        w["l0.shift"].zero_()
        w["embed"][:, DIRECTION] = 0.0
        w["embed"][NEEDLE, DIRECTION] = 6.0                      # the norm's tanh saturates: a ≈ ±1 there for the needle only
        w["l0.norm1"][DIRECTION] = 1.0
        w["l0.norm1.b"][DIRECTION] = 0.0
        for name in ("l0.mix.q", "l0.mix.k", "l0.mix.v"):
            w[name][:, DIRECTION] = 0.0
        j = dim - 1                                               # a dim that is not rotated
        w["l0.mix.k"][j, DIRECTION] = 4.0                         # map 1 of the kv head
        w["l0.mix.k.b"][j] = 0.0
        for h in range(2):
            w["l0.mix.q.b"][h * 2 * dim + j] = 6.0                # every query looks for it
        w["l0.mix.v"][:, DIRECTION] = 3.0                         # and its value stands out

    return cfg, patch


@pytest.mark.parametrize("window,keep", [(20, 3), (70, 0), (64, 64), (130, 5)])
def test_a_key_just_inside_and_just_outside_the_window_and_the_kept_tokens(tmp_path, window, keep):
    cfg, patch = needle_model(tmp_path, window, keep)
    pcfg, w = make(cfg, tmp_path, seed=21, std=0.05, norm_std=0.0, patch=patch)
    T = 200
    base = [t if t != NEEDLE else NEEDLE + 1 for t in tiny.random_prompt(64, T, 99)]
    places = [T - 1 - (window - 1), T - 1 - window, T - 2 - (window - 1), 0, 63, 64]
    if keep:
        places += [keep - 1, keep]
    engines = {dt: Engine.from_folder(str(tmp_path), dtype=dt, max_tokens=64 * 4, max_seqs=1) for dt in ("float32", "bfloat16")}
    last = {}
    for place in places:
        toks = list(base)
        toks[place] = NEEDLE
        ref = D.model_logits(pcfg, w, toks)
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
    # the test can see the edges: a needle inside changes the last logits by far more than the tolerance
    inside, outside = last[T - 1 - (window - 1)], last[T - 1 - window]
    assert float((inside - outside).abs().max() / inside.abs().max()) > 0.2
    if keep:
        assert float((last[keep - 1] - last[keep]).abs().max() / last[keep - 1].abs().max()) > 0.2


def test_a_far_key_among_hundreds_without_a_window(tmp_path):
    cfg, patch = needle_model(tmp_path, None, 0)
    pcfg, w = make(cfg, tmp_path, seed=22, std=0.05, norm_std=0.0, patch=patch)
    T = 700
    base = [t if t != NEEDLE else NEEDLE + 1 for t in tiny.random_prompt(64, T, 5)]
    plain_last = D.model_logits(pcfg, w, base)[-1]
    eng = Engine.from_folder(str(tmp_path), dtype="float32", max_tokens=64 * 11, max_seqs=1)
    for place in (1, 64, 383, 640):
        toks = list(base)
        toks[place] = NEEDLE
        ref = D.model_logits(pcfg, w, toks)
        assert float((ref[-1] - plain_last).abs().max() / ref[-1].abs().max()) > 0.2
        s = eng.acquire()
        head = eng.step([(s, toks[:-1], [T - 2])]).cpu()
        tail = eng.step([(s, [toks[-1]], [0])]).cpu()
        eng.release(s)
        assert worst(head[0], ref[-2]) <= 2e-5 and worst(tail[0], ref[-1]) <= 2e-5, place


# ---------------------------------------------------------------------------------------------- generation, the program
@pytest.mark.parametrize("name", ["a", "c"])
def test_greedy_generation_through_the_entry_point(models, name):
    m = models[name]
    prompts = [tiny.random_prompt(m.vocab, n, 7 * n) for n in (1, 9, 70, 30)]
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 8, max_seqs=3)     # two batches
    results, metrics = engine.generate(prompts, 12, SamplingParams(), stop_ids=[])
    for p, r in zip(prompts, results):
        ids = list(p)
        for tok in r.tokens:                                   # along the engine's own tokens: the chosen one is the largest
            row = D.model_logits(m.cfg, m.w, ids)[-1]
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
    compare(traces.collect(steps, str(out), m.vocab), refs_of(m, reqs), 3e-2, "trace program")


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
    assert line["tokens"] == D.generate_greedy(m.cfg, m.w, prompt, 5) and line["finish_reason"] == "length"
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["a"]))
    proc = subprocess.run([sys.executable, exe, "generate", "--random", str(cfg_file), "--token-ids", "1,2,3",
                           "--token-ids", "9,8,7,6,5", "--max-new-tokens", "4", "--temp", "0.7", "--seed", "2", "--ctx", "128"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(x) for x in proc.stdout.strip().splitlines()]
    assert [len(x["tokens"]) for x in lines] == [4, 4]


def test_trace_budget_counts_tokens_and_many_short_requests_fit(models, tmp_path):
    """The trace program's --max-tokens is a count of tokens without padding: a dozen live requests of a few tokens
    each need a page apiece although together they hold less than two pages' worth."""
    m = models["d"]
    reqs = {f"s{i}": tiny.random_prompt(m.vocab, 3 + i, 50 + i) for i in range(12)}
    steps = traces.ragged_batches(reqs, 12, {rid: 2 for rid in reqs})
    peak = sum(len(t) for t in reqs.values())
    assert peak < 2 * 64 * 2
    out = tmp_path / "out"
    traces.run_in_process(m.folder, "float32", steps, str(out), max_tokens=peak)
    compare(traces.collect(steps, str(out), m.vocab), refs_of(m, reqs), 2e-5, "many short requests")
