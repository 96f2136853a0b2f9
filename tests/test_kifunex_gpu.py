"""The Kifunex decoder and its mechanisms against the plain implementation (tests/plain_kifunex.py): every part
alone, then whole models through the engine's step function, cache manager and scheduler, for every way of cutting
the work into steps.  The configurations are small and of this file's own making; weights are random, and where
random weights would hide a fault (a window's edge, a far key) they are shaped so that it shows."""
import json
import math

import pytest
import torch

import plain_kifunex as pk

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64

SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
CONFIGS = {
    # two windows (two groups of pages), a layer without a feed-forward, two layers that run with earlier layers'
    # tensors, three copies of the stream, part of a head turned with scaling, a shared expert of its own width
    "M": pk.model_config(
        [pk.attention_layer(dim=32, heads=4, kv_heads=2, window=24, rot_dims=16, scaling=SCALING, scale=0.2,
                            mlp=pk.moe(experts=6, top=2, ff=24, shared_ff=40, scale=1.25)),
         pk.attention_layer(dim=48, heads=3, kv_heads=3, window=17, rot_dims=48, base=500.0, scale=0.11, mlp=None),
         pk.attention_layer(dim=32, heads=4, kv_heads=2, window=24, rot_dims=16, scaling=SCALING, scale=0.2,
                            mlp=pk.moe(experts=6, top=2, ff=24, shared_ff=40, scale=1.25), weights_of=0),
         pk.attention_layer(dim=48, heads=3, kv_heads=3, window=17, rot_dims=48, base=500.0, scale=0.11, mlp=None,
                            weights_of=1)],
        width=96, vocab=210, streams=3, logit_scale=1.5, logit_softcap=9.0),
    # one copy of the stream, no cap and no scale on the logits, one expert per token, no shared expert, nothing
    # turned in one layer, a window longer than any request, a head size that is no multiple of sixteen, a shared
    # expert that is two experts wide
    "N": pk.model_config(
        [pk.attention_layer(dim=40, heads=2, kv_heads=1, window=500, rot_dims=0, scale=0.3,
                            mlp=pk.moe(experts=4, top=1, ff=32, shared_ff=0, scale=2.0)),
         pk.attention_layer(dim=64, heads=4, kv_heads=1, window=33, rot_dims=32, base=10000.0, scale=0.15,
                            mlp=pk.moe(experts=5, top=3, ff=16, shared_ff=32, scale=0.7))],
        width=64, vocab=130, streams=1, logit_scale=1.0, logit_softcap=0.0),
}
SEEDS = {"M": 3, "N": 5}
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
# A bfloat16 run may rightly choose another expert than the float64 run where the last chosen and the first left-out
# choice scores are this close; such a row may exceed the tolerance, and only a few rows are such rows.
EDGE, MAX_EDGE_SHARE = 0.005, 0.1


def ids_for(name, n, salt=0):
    g = torch.Generator().manual_seed(2000 + 31 * n + salt + ord(name))
    return [int(t) for t in torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g)]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        W = pk.make_weights(cfg, SEEDS[name])
        out[name] = (cfg, W, pk.write_folder(cfg, W, str(tmp_path_factory.mktemp("kif_" + name))))
    return out


_plain = {}


def plain_logits(models, name, ids):
    """(logits, per row the smallest router margin of any layer)"""
    key = (name, tuple(ids))
    if key not in _plain:
        cfg, W, _ = models[name]
        margins = []
        lg = pk.forward(cfg, W, ids, margins=margins)
        _plain[key] = (lg, torch.stack(margins).min(dim=0).values if margins else torch.full((len(ids),), math.inf))
    return _plain[key]


def close(got, want, rel, what, margins=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    err = (got - want).abs().reshape(got.shape[0], -1).max(dim=1).values
    bound = rel * max(1e-3, float(want.abs().max()))
    bad = err > bound
    if margins is not None:
        edge = margins < EDGE
        assert int(edge.sum()) <= max(4, MAX_EDGE_SHARE * len(edge)), f"{what}: too many rows on a router's edge"
        bad = bad & ~_after(edge)
    if bool(bad.any()):
        row = int(torch.nonzero(bad)[0])
        raise AssertionError(f"{what}: error {float(err[row]):.3g} > {bound:.3g} at row {row} (first of {int(bad.sum())})")


def _after(edge):
    """Rows that an edge row can reach: the keys are the values, so a row that took another expert changes what
    every later row of its window reads.  All rows from the first edge row on."""
    out = edge.clone()
    if bool(edge.any()):
        out[int(torch.nonzero(edge)[0]):] = True
    return out


def make_runner(folder, dtype, max_tokens, max_requests=4, **kw):
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    return ModelRunner(folder, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, **kw)


class Steps:
    """Feeds requests through ``ModelRunner.step`` and keeps the logits per (request, position)."""

    def __init__(self, runner):
        from nano_vllm_cpp_b200.engine.batch import StepEntry
        self.runner, self.StepEntry, self.fed, self.logits = runner, StepEntry, {}, {}

    def step(self, parts, end=()):
        entries = [self.StepEntry(rid, list(toks), list(range(len(toks)))) for rid, toks in parts]
        out = self.runner.step(entries).float().cpu()
        r = 0
        for e in entries:
            base = self.fed.get(e.rid, 0)
            for w in e.want:
                self.logits[(e.rid, base + w)] = out[r]
                r += 1
            self.fed[e.rid] = base + len(e.tokens)
        for rid in end:
            self.runner.close(rid)
            self.fed.pop(rid, None)
        self.runner.manager.check()

    def rows(self, rid, n):
        return torch.stack([self.logits[(rid, p)] for p in range(n)])


def check_rows(st, models, name, rid, ids, dtype, what):
    want, margins = plain_logits(models, name, ids)
    close(st.rows(rid, len(ids)), want, TOL[dtype], what, margins if dtype == "bfloat16" else None)


# ------------------------------------------------------------------------------- the parts alone
def ctx_for(dtype, fast=True):
    from nano_vllm_cpp_b200.csrc import ops
    from nano_vllm_cpp_b200.parts import RunContext
    return RunContext(device=torch.device(DEV), act_dtype=dtype, err=ops.ErrorFlag(DEV), page_size=16, fast_kernels=fast)


class Fetch:
    def __init__(self, tensors, prefix, dtype):
        self.t, self.p, self.dtype = tensors, prefix, dtype

    def __call__(self, name):
        t = self.t[self.p + name]
        return t.to(torch.float32 if t.dim() <= 1 else self.dtype).to(DEV)

    def has(self, name):
        return (self.p + name) in self.t


@pytest.mark.parametrize("H", [64, 50, 256, 1100])
@pytest.mark.parametrize("S", [1, 2, 3, 8])
def test_copies_of_the_stream_alone(S, H):
    """One launch brings the copies up to date, reads them and norms what it read: with a dense pending output,
    with a weighted sum of rows that has not been taken yet, with nothing pending, and the closing sum."""
    from nano_vllm_cpp_b200.csrc import ops
    g = torch.Generator().manual_seed(7 * S + H)
    T, R, P = 9, 5, 23
    X = torch.randn(T, S, H, generator=g, dtype=F64)
    y = torch.randn(T, H, generator=g, dtype=F64)
    M = torch.eye(S, dtype=F64) + 0.3 * torch.randn(S, S, generator=g, dtype=F64)
    w, r = torch.randn(S, generator=g, dtype=F64), torch.randn(S, generator=g, dtype=F64)
    alpha = torch.tensor([0.7], dtype=F64)
    gain, shift = 1 + 0.2 * torch.randn(H, generator=g, dtype=F64), 0.1 * torch.randn(H, generator=g, dtype=F64)
    dev = lambda t: t.float().to(DEV).contiguous()
    norm = (dev(alpha), dev(gain), dev(shift))
    # a dense pending output
    x = dev(X.reshape(T, S * H))
    out, out32 = torch.empty(T, H, dtype=torch.bfloat16, device=DEV), torch.empty(T, H, dtype=torch.float32, device=DEV)
    ops.stream_mix_norm(x, S, branch=dev(y), carry=dev(M), write=dev(w), read=dev(r), norm=norm, out=out, out32=out32)
    Xn = torch.einsum("cd,tcw->tdw", M, X) + w[None, :, None] * y[:, None, :]
    u = torch.einsum("c,tcw->tw", r, Xn)
    close(x.view(T, S, H), Xn, 1e-6, "copies after a dense output")
    close(out32, pk.dyt(u, alpha, gain, shift), 1e-5, "normed rows")
    close(out, pk.dyt(u, alpha, gain, shift), 2 ** -7, "normed rows, bfloat16")
    # a sum of rows that has not been taken, with a dense term; read without a norm
    rows, dense = torch.randn(P, H, generator=g, dtype=F64), torch.randn(T, H, generator=g, dtype=F64)
    index = torch.randint(0, P, (T, R), generator=g)
    weight = torch.randn(T, R, generator=g, dtype=F64)
    y2 = dense + torch.einsum("tr,trw->tw", weight, rows[index])
    x = dev(X.reshape(T, S * H))
    ops.stream_mix_norm(x, S, mix=(dev(rows), index.int().to(DEV), dev(weight), dev(dense), None), carry=dev(M),
                        write=dev(w), read=dev(r), out32=out32)
    Xn = torch.einsum("cd,tcw->tdw", M, X) + w[None, :, None] * y2[:, None, :]
    close(x.view(T, S, H), Xn, 1e-5, "copies after a sum of rows")
    close(out32, torch.einsum("c,tcw->tw", r, Xn), 1e-5, "what was read, without a norm")
    # nothing pending; the closing sum of the copies
    x = dev(X.reshape(T, S * H))
    ops.stream_mix_norm(x, S, read=None, norm=norm, out32=out32)
    close(x.view(T, S, H), X.float(), 0.0, "copies with nothing pending")
    close(out32, pk.dyt(X.sum(dim=1), alpha, gain, shift), 1e-5, "the closing sum")


def test_dynamic_tanh_as_an_ordinary_norm():
    """With one copy and no link the part is a norm like the others: ``x += branch`` and the normed rows."""
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    g = torch.Generator().manual_seed(11)
    T, H = 6, 72
    W = {"n": 1 + 0.2 * torch.randn(H, generator=g, dtype=F64), "n.b": 0.1 * torch.randn(H, generator=g, dtype=F64),
         "n.alpha": torch.tensor(1.3, dtype=F64)}
    norm = build_part("norm", PartSpec("dynamic_tanh", dict(size=H, weight_name="n", shift_name="n.b", alpha_name="n.alpha")))
    norm.load(Fetch(W, "", torch.bfloat16), ctx_for(torch.bfloat16))
    X, y = torch.randn(T, H, generator=g, dtype=F64), torch.randn(T, H, generator=g, dtype=F64)
    x = X.float().to(DEV)
    h, h32 = norm.forward(x, y.float().to(DEV), want_f32=True)
    close(x, X + y, 1e-6, "stream")
    close(h32, pk.dyt(X + y, W["n.alpha"], W["n"], W["n.b"]), 1e-5, "rows")
    assert h.dtype == torch.bfloat16
    close(h, h32, 2 ** -7, "bfloat16 rows")


def test_scaled_and_capped_logits():
    from nano_vllm_cpp_b200.csrc import ops
    z = torch.randn(5, 77, generator=torch.Generator().manual_seed(12), dtype=F64) * 20
    for scale, cap in ((1.7, 11.0), (0.5, 0.0), (1.0, 3.0)):
        got = z.float().to(DEV)
        ops.scale_softcap(got, scale, cap)
        close(got, cap * torch.tanh(z * scale / cap) if cap > 0 else z * scale, 1e-6, f"scale {scale} cap {cap}")


def run_cut(part, cache, xs, cuts, dtype, tables, ctx, slots=None):
    """``xs``: one [T_i, width] input per request; ``cuts``: per step, the rows every request runs ((lo, hi) or
    None).  Returns per request the float32 outputs of all its rows."""
    from nano_vllm_cpp_b200.engine.batch import StepEntry, EntryInfo
    from batch_builder import build_batch
    outs = [[] for _ in xs]
    slots = slots or list(range(len(xs)))
    width = max(len(t) for t in tables)
    for cut in cuts:
        ses, infos, tabs, rows, who, row0 = [], [], [], [], [], 0
        for i, c in enumerate(cut):
            if c is None:
                continue
            lo, hi = c
            ses.append(StepEntry(i, [0] * (hi - lo), []))
            infos.append(EntryInfo(i, slots[i], lo, hi - lo, row0))
            tabs.append(tables[i])
            rows.append(xs[i][lo:hi])
            who.append((i, hi - lo))
            row0 += hi - lo
        batch = build_batch(ses, infos, [tabs], width, DEV)
        h = torch.cat(rows).to(dtype).to(DEV)
        y = part.forward(h, batch, cache.view(0))
        ctx.err.check("part")
        at = 0
        for i, n in who:
            outs[i].append(y[at:at + n].float().cpu())
            at += n
    return [torch.cat(o) for o in outs]


def attention_setup(m, width, W, dtype, fast=True, pages=48):
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    from nano_vllm_cpp_b200.cache import DeviceCache
    rot = m.get("rot") or {"dims": 0}
    position = PartSpec("none") if not rot["dims"] else PartSpec("rotary_neox", dict(
        rotary_dim=rot["dims"], theta=rot["base"], scaling=rot.get("scaling")))
    part = build_part("mixer", PartSpec("paged_attention", dict(
        hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], bias=False,
        window=m["mask"]["size"] if m.get("mask") else 0, scale=m["scale"], values_from_keys=True, exact_weights=True,
        position=position, names={"q": "q", "k": "k", "o": "o"})))
    ctx = ctx_for(dtype, fast)
    part.load(Fetch(W, "m.", dtype), ctx)
    cache = DeviceCache([part.cache_spec()], 16, 4, DEV, dtype)
    cache.allocate(pages, 48)
    return part, cache, ctx


def attention_weights(m, width, seed, scale=1.0):
    cfg = pk.model_config([{"type": "attention", "mixer": m, "mlp": None}], width=width, vocab=8)
    W = pk.make_weights(cfg, seed, scale)
    return {k.replace("l0.mix.", "m."): v for k, v in W.items() if k.startswith("l0.mix.")}


def inputs(width, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(torch.bfloat16).double() for n in lengths]


MIXERS = [pk.attention_layer(dim=32, heads=4, kv_heads=2, window=24, rot_dims=16, scaling=SCALING, scale=0.2)["mixer"],
          pk.attention_layer(dim=48, heads=3, kv_heads=3, window=17, rot_dims=48, base=500.0, scale=0.11)["mixer"],
          pk.attention_layer(dim=64, heads=8, kv_heads=1, window=44, rot_dims=0, scale=0.125)["mixer"],
          pk.attention_layer(dim=40, heads=2, kv_heads=1, window=1, rot_dims=20, scale=0.3)["mixer"],
          pk.attention_layer(dim=128, heads=2, kv_heads=2, window=64, rot_dims=64, scale=0.09)["mixer"],
          pk.attention_layer(dim=64, heads=20, kv_heads=1, window=30, rot_dims=32, scale=0.12)["mixer"],
          pk.attention_layer(dim=192, heads=2, kv_heads=1, window=50, rot_dims=96, scaling=SCALING, scale=0.07)["mixer"],
          pk.attention_layer(dim=96, heads=3, kv_heads=1, window=21, rot_dims=48, scale=0.1)["mixer"],
          pk.attention_layer(dim=256, heads=1, kv_heads=1, window=35, rot_dims=256, scale=0.06)["mixer"]]
CUTS = [[(0, 37), (0, 2)], [(37, 38), (2, 19)], [(38, 40), (19, 20)], [(40, 41), (20, 21)], [None, (21, 50)],
        [(41, 64), (50, 51)], [(64, 65), None], [(65, 66), None]]
PAGES = [[7, 3, 11, 0, 9], [5, 2, 8, 10]]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", MIXERS)
def test_attention_alone(dtype, m, fast):
    """Two requests on scattered pages, in portions beside single rows: grouped heads, windows shorter and longer
    than a page, part of a head turned, nothing turned, a window of one."""
    width = 80
    W = attention_weights(m, width, 21)
    part, cache, ctx = attention_setup(m, width, W, dtype, fast)
    xs = inputs(width, [66, 51], 22)
    got = run_cut(part, cache, xs, CUTS, dtype, PAGES, ctx)
    for i, x in enumerate(xs):
        close(got[i], pk.window_attention(x, W, "m.", m), 1e-4 if dtype == torch.float32 else 3e-2, f"request {i}")


def edge_case(window, T, i, j, width=64):
    """Weights and inputs for which row i's softmax falls in halves on key j and on itself: q heads are copies of the
    k head (nothing is turned), so a score is a product of two keys; row i's key is large, row j's is the same plus an
    equally large part at right angles to it (the same score, another value), and the other rows are small."""
    m = pk.attention_layer(dim=32, heads=2, kv_heads=1, window=window, rot_dims=0, scale=1.0)["mixer"]
    m["rot"] = None
    W = attention_weights(m, width, 31)
    W["m.q"] = torch.cat([W["m.k"], W["m.k"]])
    g = torch.Generator().manual_seed(32)
    x = 0.05 * torch.randn(T, width, generator=g, dtype=F64)
    big, side = torch.randn(width, generator=g, dtype=F64), torch.randn(width, generator=g, dtype=F64)
    kb, ks = W["m.k"] @ big, W["m.k"] @ side
    side = side - big * float(ks @ kb) / float(kb @ kb)
    big, side = big * (2.5 / float(kb.norm())), side * (2.5 / float((W["m.k"] @ side).norm()))
    x[i], x[j] = big, big + side
    return m, W, x.to(torch.bfloat16).double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window,i,gap", [(24, 50, 23), (24, 50, 24), (16, 47, 15), (16, 47, 16), (17, 33, 16), (17, 33, 17),
                                          (400, 330, 327), (400, 330, 17), (300, 650, 299), (300, 650, 300)])
def test_one_key_stands_out(window, i, gap, decoded, dtype):
    """A key just inside the window (gap = window - 1) takes half of row i's weight, a key just outside it
    (gap = window) takes none; at page borders, in a prompt and when row i is decoded alone after single rows; and a
    key hundreds of positions back among scattered pages."""
    T = i + 3
    m, W, x = edge_case(window, T, i, i - gap)
    part, cache, ctx = attention_setup(m, 64, W, dtype)
    table = [(5 * p + 3) % 47 for p in range((T + 15) // 16)]
    assert len(set(table)) == len(table)
    cuts = [[(0, T)]] if not decoded else [[(0, i - 2)]] + [[(t, t + 1)] for t in range(i - 2, T)]
    got = run_cut(part, cache, [x], cuts, dtype, [table], ctx)[0]
    want = pk.window_attention(x, W, "m.", m)
    close(got, want, 1e-4 if dtype == torch.float32 else 3e-2, "rows")
    # the case shows what it is meant to show: with and without key j row i differs by much more than the tolerance
    other = pk.window_attention(x, W, "m.", dict(m, mask={"size": gap if gap < window else gap + 1}))
    assert float((other[i] - want[i]).abs().max()) > 0.2 * float(want.abs().max())


@pytest.mark.parametrize("D", [64, 128])
def test_softmax_weights_keep_their_bits_in_the_product_with_the_values(D):
    """Values of alternating sign and large size under nearly equal weights: the sum cancels, and weights rounded to
    bfloat16 would show in it (the test computes that they would, on a third of the values); the three-term kernels
    for prompts (tcgen05 and mma.sync) and the decode kernel's float32-weights form stay inside the rounding of
    their bfloat16 output."""
    from nano_vllm_cpp_b200.csrc import ops
    T, Hq, page, scale = 200, 2, 16, D ** -0.5
    g = torch.Generator().manual_seed(5)
    q = (0.3 * torch.randn(T, Hq, D, generator=g)).to(torch.bfloat16)
    k = torch.randn(T, D, generator=g).to(torch.bfloat16)
    sign = torch.tensor([1.0 if j % 2 == 0 else -1.0 for j in range(T)])
    v = (sign[:, None] * 48.0 + torch.randn(T, D, generator=g)).to(torch.bfloat16)
    s = torch.einsum("thd,jd->htj", q.double(), k.double()) * scale
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), -1e30)
    ref = torch.einsum("htj,jd->thd", torch.softmax(s, dim=2), v.double())
    bound = 2 ** -8 * ref.abs() + 2e-3
    e = torch.exp(s - s.max(dim=2, keepdim=True).values)
    rounded = torch.einsum("htj,jd->thd", e.float().to(torch.bfloat16).double() / e.sum(dim=2, keepdim=True), v.double())
    assert float(((rounded - ref).abs() > bound)[20:].float().mean()) > 0.2       # the case shows what it is meant to
    n_pages = (T + page - 1) // page
    table = [(7 * i + 2) % 29 for i in range(n_pages)]
    kc = torch.zeros(29, 1, page, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    for i, pg in enumerate(table):
        n = min(page, T - i * page)
        kc[pg, 0, :n] = k[i * page:i * page + n].to(DEV)
        vc[pg, 0, :n] = v[i * page:i * page + n].to(DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    bt = torch.tensor([table], **i32)
    qd = q.reshape(T, Hq * D).to(DEV).contiguous()
    err = ops.ErrorFlag(DEV)
    tiles = T // ops.attention_prefill_tile_rows() + 1
    for kernel in ("auto", "mma"):
        out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill(qd, kc, vc, bt, torch.tensor([0, T], **i32), torch.tensor([0], **i32), tiles, scale, 0, out,
                              Hq, 1, D, err=err, kernel=kernel, weight_terms=3)
        err.check(kernel)
        worst = float(((out.double().cpu().view(T, Hq, D) - ref).abs() / bound).max())
        assert worst <= 1.0, f"{kernel}: {worst:.2f} times the bound"
    rows = list(range(T - 5, T))
    out = torch.zeros(len(rows), Hq * D, dtype=torch.bfloat16, device=DEV)
    for splits_ctx in (T, 4096):                   # (the longest context fixes the number of key splits)
        ops.attention_decode(qd[rows].contiguous(), kc, vc, bt.repeat(len(rows), 1).contiguous(),
                             torch.arange(len(rows), **i32), torch.tensor(rows, **i32), scale, 0, out, Hq, 1, D, splits_ctx,
                             err=err, float_weights=True)
        err.check("decode")
        worst = float(((out.double().cpu().view(len(rows), Hq, D) - ref[rows]).abs() / bound[rows]).max())
        assert worst <= 1.0, f"decode: {worst:.2f} times the bound"


def route_case(E, K, T, seed, spread):
    g = torch.Generator().manual_seed(seed)
    W = {"m.router": torch.randn(E, 48, generator=g, dtype=F64) / 4, "m.correction": spread * torch.randn(E, generator=g, dtype=F64)}
    h = torch.randn(T, 48, generator=g, dtype=F64)
    return W, h


@pytest.mark.parametrize("E,K,spread", [(6, 2, 0.3), (8, 3, 3.0), (5, 5, 0.5), (1, 1, 0.0), (70, 4, 1.0), (8, 1, 0.3)])
def test_router_alone(E, K, spread):
    """Sigmoid scores, the choice by score plus correction (corrections large enough to change the choice and to
    make choice scores negative), weights without it times the scale; both routing kernels; with an always-on
    chunk behind the chosen experts, which weighs one."""
    from nano_vllm_cpp_b200.csrc import ops
    for T in (1, 7, 300):
        W, h = route_case(E, K, T, 40 + E + T, spread)
        r = {"experts": E, "top": K, "scale": 1.75}
        picks, _ = pk.route(h, W, "m.", r)
        logits = (h @ W["m.router"].T).float().to(DEV)
        rule = ("sigmoid", W["m.correction"].float().to(DEV), 1.75)
        for C in (0, 1):
            idx = torch.empty(T, K + C, dtype=torch.int32, device=DEV)
            score = torch.empty(T, K + C, dtype=torch.float32, device=DEV)
            kinds = ["topk"] + (["small"] if ops.moe_route_small_usable(T, E, K, C, 48) else [])
            for kind in kinds:
                idx.fill_(-1)
                if kind == "topk":
                    ops.router_topk(logits, K, False, idx, score, C, None, rule=rule)
                else:
                    al = ops.MoeAlignment(T * (K + C), E + C, 16, DEV, 0)
                    ops.moe_route_small(logits, K, False, C, None, idx, score, al, ops.ErrorFlag(DEV), rule=rule)
                gi, gs = idx.cpu(), score.cpu().double()
                for t in range(T):
                    assert [int(e) for e in gi[t, :K]] == [e for e, _ in picks[t]], f"{kind} row {t}"
                    assert max(abs(float(gs[t, k]) - picks[t][k][1]) for k in range(K)) < 1e-5
                    if C:
                        assert int(gi[t, K]) == E and float(gs[t, K]) == 1.0


MLPS = [pk.moe(experts=6, top=2, ff=24, shared_ff=24, scale=1.25), pk.moe(experts=5, top=5, ff=40, shared_ff=16, scale=0.5),
        pk.moe(experts=8, top=1, ff=32, shared_ff=0, scale=2.0), pk.moe(experts=4, top=3, ff=16, shared_ff=32, scale=1.0),
        pk.moe(experts=3, top=2, ff=20, shared_ff=12, scale=1.0),
        dict(pk.moe(experts=16, top=4, ff=128, shared_ff=256, scale=1.5), width=256),      # sizes the tensor-core products take
        dict(pk.moe(experts=12, top=3, ff=64, shared_ff=64, scale=0.8), width=128)]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mlp", MLPS)
def test_mixture_alone(dtype, mlp, fast):
    """The feed-forward with one row, a handful, and more rows than the one-launch routing takes; a shared expert as
    wide as an expert, twice as wide, of a width of its own, and none; widths the tensor-core product refuses."""
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    mlp = dict(mlp)
    width = mlp.pop("width", 64)
    cfg = pk.model_config([pk.attention_layer(mlp=mlp)], width=width, vocab=8)
    W = {k.replace("l0.mlp.", "m."): v for k, v in pk.make_weights(cfg, 51).items() if k.startswith("l0.mlp.")}
    ff = build_part("feed_forward", PartSpec("sparse_moe_swiglu", dict(
        hidden_size=width, num_experts=mlp["router"]["experts"], top_k=mlp["router"]["top"],
        intermediate_size=mlp["expert"]["ff"], shared_intermediate_size=mlp["shared"]["ff"] if mlp["shared"] else 0,
        score="sigmoid", route_scale=mlp["router"]["scale"], choice_bias=True, shared_gate=False,
        names={"router": "router", "correction": "correction", "expert_gate": "e{}.gate", "expert_up": "e{}.up",
               "expert_down": "e{}.down", "shared_gate_proj": "shared.gate", "shared_up": "shared.up",
               "shared_down": "shared.down"})))
    ff.load(Fetch(W, "m.", dtype), ctx_for(dtype, fast))
    for T in (1, 5, 70, 300):
        x = inputs(width, [T], 52 + T)[0]
        margins = []
        want = pk.mixture(x, W, "m.", mlp, margins)
        h32 = x.float().to(DEV)
        y = ff.forward(h32.to(dtype), h32, None)
        y = y.sum() if hasattr(y, "sum") and not isinstance(y, torch.Tensor) else y
        # (the router reads float32 rows here, so only a float32 tie could change a choice)
        close(y, want, 1e-4 if dtype == torch.float32 else 3e-2, f"T={T}")


# ------------------------------------------------------------------------------- whole models through the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M", "N"])
def test_whole_prompts(name, dtype, models):
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    for n in (1, 2, 3, 17, 64, 65, 150):
        ids = ids_for(name, n)
        st.step([(f"w{n}", ids)], end=[f"w{n}"])
        check_rows(st, models, name, f"w{n}", ids, dtype, f"{name} whole n={n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M", "N"])
def test_prompt_then_token_by_token(name, dtype, models):
    """A short prompt in one step, then ninety rows one at a time (the windows pass over decoded tokens; pages of
    positions that fell out of every window go back; steps of the same shape are replayed from a captured graph),
    and a sequence that is decoded from its first token on."""
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    ids = ids_for(name, 100, salt=1)
    st.step([("d", ids[:10])])
    for t in range(10, 100):
        st.step([("d", ids[t:t + 1])])
    check_rows(st, models, name, "d", ids, dtype, f"{name} decode")
    st.step([], end=["d"])
    ids = ids_for(name, 20, salt=2)
    for t in range(20):
        st.step([("e", ids[t:t + 1])])
    check_rows(st, models, name, "e", ids, dtype, f"{name} decode from the first token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M", "N"])
def test_portions_of_several_sizes(name, dtype, models):
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    ids = ids_for(name, 131, salt=3)
    sizes = [2, 1, 2, 14, 13, 3, 2, 30, 1, 1, 17, 2, 33, 10]
    assert sum(sizes) == 131
    at = 0
    for s in sizes:
        st.step([("p", ids[at:at + s])])
        at += s
    check_rows(st, models, name, "p", ids, dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M", "N"])
def test_unequal_requests_together_with_pages_used_again(name, dtype, models):
    """Three slots and 192 tokens of pages for six requests that need more in turn: portions of some beside single
    rows of others; a finished request's pages go to the next one.  Every request's logits equal those of the
    request alone."""
    runner = make_runner(models[name][2], dtype, 192, max_requests=3)
    st = Steps(runner)
    L = {"a": 50, "b": 37, "c": 64, "d": 20, "e": 61, "f": 33}
    ids = {r: ids_for(name, n, salt=ord(r)) for r, n in L.items()}
    at = {r: 0 for r in L}

    def take(r, n):
        toks = ids[r][at[r]:at[r] + n]
        at[r] += len(toks)
        return (r, toks)

    def done(*rs):
        return [r for r in rs if at[r] == L[r]]

    st.step([take("a", 30), take("b", 2)])
    st.step([take("a", 1), take("b", 35), take("c", 3)], end=done("b"))
    st.step([take("a", 19), take("c", 1), take("d", 20)], end=done("a", "d"))
    st.step([take("c", 60), take("e", 2), take("f", 1)], end=done("c"))
    st.step([take("e", 1), take("f", 2)])
    st.step([take("e", 58), take("f", 30)], end=done("e", "f"))
    for r, n in L.items():
        assert at[r] == n
        check_rows(st, models, name, r, ids[r], dtype, f"{name} request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_a_row(dtype, models):
    """The same request whole, in portions and beside another request: float32 rows agree to rounding of sums
    (the products of a one-row step take another kernel), bfloat16 rows to bfloat16 rounding."""
    name = "M"
    ids = ids_for(name, 70, salt=9)
    other = ids_for(name, 40, salt=10)
    _, margins = plain_logits(models, name, ids)
    runs = []
    for cut in ([70], [33, 1, 2, 34], [64, 6]):
        runner = make_runner(models[name][2], dtype, 256)
        st = Steps(runner)
        at = 0
        for k, s in enumerate(cut):
            st.step([("x", ids[at:at + s])] + ([("o", other[:20] if k == 0 else other[20 + k:21 + k])] if len(cut) == 4 else []))
            at += s
        runs.append(st.rows("x", 70))
    for r in runs[1:]:
        close(r, runs[0], 2e-5 if dtype == "float32" else 3e-2, "the same rows cut another way",
              margins if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype, models):
    """The engine's own entry point, scheduler and sampling: greedy tokens follow the plain implementation's up
    to the first position where its two best logits are closer than the tolerance."""
    from nano_vllm_cpp_b200 import LLMEngine, SamplingParams
    name = "M"
    cfg, W, folder = models[name]
    prompts = [ids_for(name, 9, salt=20), ids_for(name, 3, salt=21), ids_for(name, 30, salt=22)]
    eng = LLMEngine(folder, max_model_len=96, num_kv_blocks=24, dtype=dtype, max_num_seqs=2, log_stats=False)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for k, tok in enumerate(o["token_ids"]):
            logits = pk.forward(cfg, W, seq)[-1]
            best = int(torch.argmax(logits))
            if best != tok:
                lead = float(logits[best] - logits[tok])
                bound = 2 * TOL[dtype] * float(logits.abs().max())
                assert lead <= bound, f"token {k} of a prompt of {len(p)}: {tok}, plain takes {best} with a lead of {lead:.3g}"
                break
            seq.append(tok)


def test_command_line_serves_the_design(models, tmp_path, capsys):
    """``nanovllm <folder> --tokens ...`` and ``nanovllm --config <json>`` (random weights) run this design as they
    run the others; the greedy tokens from the folder are the plain implementation's."""
    from nano_vllm_cpp_b200 import cli
    name = "N"
    cfg, W, folder = models[name]
    prompt = ids_for(name, 7, salt=30)
    rc = cli.main([folder, "--tokens", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                   "--dtype", "float32", "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0, out
    toks = [int(t) for t in out.strip().splitlines()[-1].split(":")[1].split()]
    assert toks == pk.greedy_generate(cfg, W, prompt, 6)
    path = tmp_path / "config.json"
    path.write_text(json.dumps(CONFIGS["M"]))
    rc = cli.main(["--config", str(path), "--seed", "4", "--tokens", "5,6,7", "--max-tokens", "4", "--temperature", "0",
                   "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0 and len(out.strip().splitlines()[-1].split(":")[1].split()) == 4
