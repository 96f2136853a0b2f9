"""The Bizodra decoder and its mechanisms against the plain implementation (tests/plain_bizodra.py): every part
alone, then whole models through the engine's step function, cache manager and scheduler, for every way of cutting
the work into steps.  The configurations are small and of this file's own making; weights are random, and where
random weights would hide a fault they are shaped so that it shows."""
import copy
import math

import pytest
import torch

import plain_bizodra as pb

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

ROT_A = {"dims": 16, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
ROT_B = {"dims": 48, "base": 500.0}
LEFT_A = {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 48, "scale": 0.3, "rot": ROT_A}
LEFT_B = {"heads": 3, "kv_heads": 3, "dim": 48, "vdim": 16, "scale": 0.2, "rot": ROT_B}
RIGHT_A = {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 3}
RIGHT_B = {"heads": 1, "kv_heads": 1, "dim": 32, "vdim": 16, "conv": 2}
LSTM_A = {"heads": 3, "dim": 16, "vdim": 24, "gate_cap": 10.0}
LSTM_B = {"heads": 1, "dim": 40, "vdim": 64, "gate_cap": 20.0}

CONFIGS = {
    # two kinds of layers in another order than any other file has, a layer without an MLP, a rotation of part of
    # the head with scaling, grouped heads on both sides, three taps
    "P": {"architecture": "Bizodra", "vocab": 210, "width": 96, "norm": {"eps": 1e-6}, "token_side": {"dim": 8},
          "layers": [{"type": "parallel", "mixer": {"left": LEFT_A, "right": RIGHT_A}, "mlp": {"kind": "dense", "ff": 160}},
                     {"type": "mlstm", "mixer": LSTM_A, "mlp": None},
                     {"type": "mlstm_2", "mixer": LSTM_B, "mlp": {"kind": "dense", "ff": 72}}]},
    # no token input, one head where the other has several, no scaling, two taps, values narrower than keys
    "Q": {"architecture": "Bizodra", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
          "layers": [{"type": "mlstm_2", "mixer": LSTM_B, "mlp": {"kind": "dense", "ff": 48}},
                     {"type": "parallel", "mixer": {"left": LEFT_B, "right": RIGHT_B}, "mlp": None},
                     {"type": "parallel", "mixer": {"left": LEFT_A, "right": RIGHT_B}, "mlp": {"kind": "dense", "ff": 96}}]},
}
SEEDS = {"P": 3, "Q": 5}
TOL = {"float32": 1e-4, "bfloat16": 4e-2}


def ids_for(name, n, salt=0):
    g = torch.Generator().manual_seed(1000 + 31 * n + salt + ord(name))
    return [int(t) for t in torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g)]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        W = pb.random_weights(cfg, SEEDS[name])
        out[name] = (cfg, W, pb.write_folder(cfg, W, str(tmp_path_factory.mktemp("biz_" + name))))
    return out


_plain = {}


def plain_logits(models, name, ids):
    key = (name, tuple(ids))
    if key not in _plain:
        cfg, W, _ = models[name]
        _plain[key] = pb.forward(cfg, W, ids)
    return _plain[key]


def close(got, want, rel, what):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    err = (got - want).abs()
    bound = rel * max(1e-3, float(want.abs().max()))
    if float(err.max()) > bound:
        row = int(err.reshape(err.shape[0], -1).max(dim=1).values.argmax())
        raise AssertionError(f"{what}: max error {float(err.max()):.3g} > {bound:.3g}, first worst row {row}")


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


# ------------------------------------------------------------------------------- the parts alone
def ctx_for(dtype, fast=True):
    from nano_vllm_cpp_b200.csrc import ops
    from nano_vllm_cpp_b200.parts import RunContext
    return RunContext(device=torch.device(DEV), act_dtype=dtype, err=ops.ErrorFlag(DEV), page_size=16, fast_kernels=fast)


class Fetch:
    def __init__(self, tensors, prefix, dtype):
        self.t, self.p, self.dtype = tensors, prefix, dtype

    def __call__(self, name):
        t = self.t[name[1:] if name.startswith("/") else self.p + name]
        return t.to(torch.float32 if (t.dim() == 1 or name.endswith(".conv")) else self.dtype).to(DEV)

    def has(self, name):
        return (self.p + name) in self.t


def run_cut(part, cache, xs, cuts, dtype, tables, ctx, slots=None, call=None):
    """``xs``: one [T_i, width] input per request; ``cuts``: per step, the rows every request runs ((lo, hi) or
    None).  Returns per request the float32 outputs of all its rows.  ``call(part, rows, batch, view)`` runs the
    part (default: a mixer's forward)."""
    from nano_vllm_cpp_b200.engine.batch import StepEntry, EntryInfo
    from batch_builder import build_batch
    outs = [[] for _ in xs]
    slots = slots or list(range(len(xs)))
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
        batch = build_batch(ses, infos, [tabs], 32, DEV)
        cache.reset_fresh(batch)
        h = torch.cat(rows).to(dtype).to(DEV)
        y = call(part, h, batch, cache.view(0)) if call else part.forward(h, batch, cache.view(0))
        ctx.err.check("part")
        at = 0
        for i, n in who:
            outs[i].append(y[at:at + n].float().cpu())
            at += n
    return [torch.cat(o) for o in outs]


CUTS = [[(0, 37), (0, 2)], [(37, 38), (2, 19)], [(38, 40), (19, 20)], [(40, 41), (20, 21)], [None, (21, 50)],
        [(41, 64), (50, 51)]]


def part_setup(kind, params, tensors, dtype, prefix="m.", fast=True):
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    from nano_vllm_cpp_b200.cache import DeviceCache
    part = build_part("mixer", PartSpec(kind, params))
    ctx = ctx_for(dtype, fast)
    part.load(Fetch(tensors, prefix, dtype), ctx)
    cache = DeviceCache([part.cache_spec()], 16, 4, DEV, dtype)
    cache.allocate(24, 32)
    return part, cache, ctx


def mixer_weights(cfg_layer, width, seed):
    cfg = {"vocab": 8, "width": width, "norm": {"eps": 1e-6}, "layers": [dict(cfg_layer, mlp=None)]}
    W = pb.random_weights(cfg, seed)
    return {k.replace("l0.mix.", "m."): v for k, v in W.items() if k.startswith("l0.mix.")}


def inputs(width, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(torch.bfloat16).double() for n in lengths]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", [LSTM_A, LSTM_B, {"heads": 2, "dim": 72, "vdim": 136, "gate_cap": 5.0},
                               {"heads": 1, "dim": 136, "vdim": 24, "gate_cap": 8.0}])
def test_matrix_lstm_alone(dtype, m, fast):
    """``fast``: the kernel that keeps a column of the matrix per thread (keys up to 128 long; beyond that, and
    without ``fast``, the kernel that keeps the matrix in shared memory)."""
    width, eps = 80, 1e-5
    W = mixer_weights({"type": "mlstm", "mixer": m}, width, 11)
    part, cache, ctx = part_setup("matrix_lstm", dict(hidden_size=width, heads=m["heads"], dim=m["dim"], vdim=m["vdim"],
                                                      gate_cap=m["gate_cap"], eps=eps), W, dtype, fast=fast)
    xs = inputs(width, [64, 51], 12)
    got = run_cut(part, cache, xs, CUTS, dtype, [[], []], ctx, slots=[2, 0])
    for i, x in enumerate(xs):
        close(got[i], pb.matrix_lstm(x, W, "m.", m, eps), TOL["float32"] if dtype == torch.float32 else 3e-2, f"request {i}")


def test_matrix_lstm_large_gates_and_first_rows():
    """Input gates far above the forget path and far below it: the running maximum starts at 0, so a first row
    whose input gate is very negative is divided by exp(-m) = 1 and not by its tiny normaliser."""
    m, width, eps = {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 30.0}, 48, 1e-6
    W = mixer_weights({"type": "mlstm", "mixer": m}, width, 13)
    W["m.i.b"] = torch.tensor([-25.0, 25.0], dtype=torch.float64)
    W["m.f.b"] = torch.tensor([6.0, -6.0], dtype=torch.float64)
    part, cache, ctx = part_setup("matrix_lstm", dict(hidden_size=width, heads=2, dim=16, vdim=24, gate_cap=30.0, eps=eps),
                                  W, torch.float32)
    xs = inputs(width, [40], 14)
    got = run_cut(part, cache, xs, [[(0, 1)], [(1, 3)], [(3, 40)]], torch.float32, [[]], ctx)
    close(got[0], pb.matrix_lstm(xs[0], W, "m.", m, eps), 1e-4, "rows")


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", [RIGHT_A, RIGHT_B, {"heads": 6, "kv_heads": 3, "dim": 40, "vdim": 72, "conv": 5},
                               {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "conv": 1},
                               {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 136, "conv": 4}])
def test_gated_delta_alone(dtype, m, fast):
    """Portions shorter than the convolution's reach (one and two rows), so that its kept inputs are a mix of old
    and new ones."""
    width, eps = 80, 1e-5
    W = mixer_weights({"type": "parallel", "mixer": {"left": LEFT_A, "right": m}}, width, 21)
    W = {k.replace("m.right.", "m."): v for k, v in W.items() if k.startswith("m.right.")}
    part, cache, ctx = part_setup("gated_delta_rule", dict(hidden_size=width, heads=m["heads"], kv_heads=m["kv_heads"],
                                                           dim=m["dim"], vdim=m["vdim"], conv=m["conv"], eps=eps), W, dtype,
                                  fast=fast)
    xs = inputs(width, [64, 51], 22)
    got = run_cut(part, cache, xs, CUTS, dtype, [[], []], ctx, slots=[1, 3])
    for i, x in enumerate(xs):
        close(got[i], pb.gated_delta(x, W, "m.", m, eps), TOL["float32"] if dtype == torch.float32 else 3e-2, f"request {i}")


def attention_part(m, width, eps, W, dtype, fast=True):
    from nano_vllm_cpp_b200.parts import PartSpec
    names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
             "q_norm": "q.norm", "k_norm": "k.norm"}
    return part_setup("paged_attention", dict(
        hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
        bias=True, out_bias=True, qk_norm_eps=eps, scale=m["scale"], sink_score=0.0, names=names,
        position=PartSpec("rotary_interleaved", dict(rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"],
                                                     scaling=m["rot"].get("scaling")))), W, dtype, fast=fast)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", [LEFT_A, LEFT_B, {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.1,
                                                "rot": {"dims": 64, "base": 1e6}}])
@pytest.mark.parametrize("fast", [True, False])
def test_sink_attention_alone(dtype, m, fast):
    """``fast`` in bfloat16: the tensor-core kernel over heads padded to one size; else the general kernel."""
    width, eps = 80, 1e-5
    W = mixer_weights({"type": "parallel", "mixer": {"left": m, "right": RIGHT_B}}, width, 31)
    W = {k.replace("m.left.", "m."): v for k, v in W.items() if k.startswith("m.left.")}
    part, cache, ctx = attention_part(m, width, eps, W, dtype, fast)
    xs = inputs(width, [64, 51], 32)
    got = run_cut(part, cache, xs, CUTS, dtype, [[7, 2, 9, 4], [0, 5, 11, 3]], ctx)
    for i, x in enumerate(xs):
        close(got[i], pb.sink_attention(x, W, "m.", m, eps), TOL["float32"] if dtype == torch.float32 else 3e-2, f"request {i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key(dtype):
    """Sharp scores (a large scale), so that every row's weight sits on few keys, somewhere among three hundred and
    across page borders: a key read from a wrong page or place changes the row.  The last rows come one at a time.
    Before that the sink: with a tiny scale every score is near 0 and the first row's only key gets weight 1/2."""
    m = {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 24, "scale": 4.0, "rot": {"dims": 32, "base": 100.0}}
    width, eps, n = 64, 1e-6, 330
    W = mixer_weights({"type": "parallel", "mixer": {"left": m, "right": RIGHT_B}}, width, 41)
    W = {k.replace("m.left.", "m."): v for k, v in W.items() if k.startswith("m.left.")}
    part, cache, ctx = attention_part(m, width, eps, W, dtype)
    xs = inputs(width, [n], 42)
    want = pb.sink_attention(xs[0], W, "m.", m, eps)
    pages = [20, 3, 17, 8, 1, 13, 0, 5, 22, 9, 11, 2, 19, 6, 15, 4, 10, 7, 21, 12, 14]
    cuts = [[(0, 15)], [(15, 17)], [(17, 300)]] + [[(t, t + 1)] for t in range(300, n)]
    got = run_cut(part, cache, xs, cuts, dtype, [pages], ctx)
    close(got[0], want, 1e-4 if dtype == torch.float32 else 4e-2, "sharp attention")
    flat = dict(m, scale=1e-4)
    part, cache, ctx = attention_part(flat, width, eps, W, dtype)
    got = run_cut(part, cache, xs, [[(0, 3)]], dtype, [pages], ctx)
    close(got[0], pb.sink_attention(xs[0][:3], W, "m.", flat, eps), 1e-4 if dtype == torch.float32 else 3e-2, "sink")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_pieces_alone(dtype):
    """The dense MLP, the token input and the branch norm with its sum, each against its formula."""
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    from nano_vllm_cpp_b200.engine.batch import StepEntry, EntryInfo
    from batch_builder import build_batch
    width, eps, T = 72, 1e-5, 19
    cfg = {"vocab": 40, "width": width, "norm": {"eps": eps}, "token_side": {"dim": 12},
           "layers": [{"type": "mlstm", "mixer": LSTM_A, "mlp": {"kind": "dense", "ff": 100}}] * 3}
    W = pb.random_weights(cfg, 51)
    ctx = ctx_for(dtype)
    x = inputs(width, [T], 52)[0]
    h = x.to(dtype).to(DEV)
    rel = 1e-5 if dtype == torch.float32 else 2e-2
    mlp = build_part("feed_forward", PartSpec("dense_mlp", dict(hidden_size=width, intermediate_size=100,
                                                                activation="gelu_erf", up_name="up", down_name="down")))
    mlp.load(Fetch(W, "l1.mlp.", dtype), ctx)
    close(mlp.forward(h, h, None), pb.dense_mlp(x, W, "l1.mlp."), rel, "mlp")
    ids = [int(t) for t in torch.randint(0, 40, (T,), generator=torch.Generator().manual_seed(53))]
    batch = build_batch([StepEntry(0, ids, [])], [EntryInfo(0, 0, 0, T, 0)], [[[0, 1]]], 4, DEV)
    side = build_part("token_input", PartSpec("gated_table", dict(hidden_size=width, vocab_size=40, dim=12, index=2, count=3,
                                                                  table_name="side.embed")))
    side.load(Fetch(W, "l2.side.", dtype), ctx)
    close(side.forward(h, batch), pb.token_input(x, torch.tensor(ids), W, "l2.side.", 2, 12), rel, "token input")
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=width, eps=eps, weight_offset=1.0, weight_name="norm1")))
    norm.load(Fetch(W, "l0.", dtype), ctx)
    g = torch.Generator().manual_seed(54)
    stream, a, b = (torch.randn(T, width, generator=g, dtype=torch.float64) for _ in range(3))
    wa, wb = (1 + 0.3 * torch.randn(width, generator=g, dtype=torch.float64) for _ in range(2))
    xs = stream.float().to(DEV)
    rows = norm.add_normed(xs, [a.float().to(DEV)])
    want = stream + pb.rms(a, eps) * (1 + W["l0.norm1"])
    close(xs, want, 1e-5, "stream after one branch")
    close(rows, want, 1e-5 if dtype == torch.float32 else 2 ** -7, "rows after one branch")
    xs = stream.float().to(DEV)
    norm.add_normed(xs, [a.float().to(DEV), b.float().to(DEV)], branch_weights=[wa.float().to(DEV), wb.float().to(DEV)],
                    mix_scale=0.5)
    mixed = 0.5 * (pb.rms(a, eps) * wa + pb.rms(b, eps) * wb)
    close(xs, stream + pb.rms(mixed, eps) * (1 + W["l0.norm1"]), 1e-5, "stream after two mixed branches")


@pytest.mark.parametrize("act", ["gelu_erf", "gelu_tanh", "silu"])
def test_activation_pass(act):
    """The activation as a pass of its own: four values per thread where the size allows, else one."""
    from nano_vllm_cpp_b200.csrc import ops
    fn = {"gelu_erf": pb.gelu_erf, "gelu_tanh": pb.gelu_tanh, "silu": pb.silu}[act]
    g = torch.Generator().manual_seed(60)
    for shape in ((7, 13), (64, 256), (3, 20)):
        z = 3 * torch.randn(shape, generator=g)
        for out_dtype, rel in ((torch.bfloat16, 2 ** -7), (torch.float32, 1e-6)):
            out = torch.empty(shape, dtype=out_dtype, device=DEV)
            ops.activation(z.to(DEV), out, act)
            close(out, fn(z.double()), rel, f"{act} {shape} {out_dtype}")


@pytest.mark.parametrize("act", ["gelu_erf", "gelu_tanh", "silu"])
def test_activation_in_the_products_epilogues(act):
    """Every product kernel applies a unary activation to its float32 sums after the bias: the one that streams the
    weights for a handful of rows, the tensor-core one (whole, with two weight tiles per block, and with K split
    and a finishing kernel), and the plain one in float32."""
    from nano_vllm_cpp_b200.csrc import ops
    fn = {"gelu_erf": pb.gelu_erf, "gelu_tanh": pb.gelu_tanh, "silu": pb.silu}[act]
    g = torch.Generator().manual_seed(61)
    K, N = 256, 328
    w = (torch.randn(N, K, generator=g) / 16).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    for M, kind in ((5, "skinny"), (300, "fast"), (2048, "fast"), (300, "split"), (37, "plain")):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        want = fn(x.double() @ w.double().T + bias.double())
        if kind == "plain":
            out = torch.empty(M, N, dtype=torch.float32, device=DEV)
            ops.gemm_plain(x.float().to(DEV), w.float().to(DEV), out, bias=bias.to(DEV), act=act)
            close(out, want, 1e-5, f"{act} plain")
            continue
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        if kind == "skinny":
            ops.skinny_gemm(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV), act=act)
        else:
            ops.gemm_fast(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV), act=act, splits=3 if kind == "split" else None)
        close(out, want, 2 ** -7, f"{act} {kind} M={M}")


# ------------------------------------------------------------------------------- whole models through the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_whole_prompts(name, dtype, models):
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    for n in (1, 2, 3, 17, 64, 65, 150):
        ids = ids_for(name, n)
        st.step([(f"w{n}", ids)], end=[f"w{n}"])
        close(st.rows(f"w{n}", n), plain_logits(models, name, ids), TOL[dtype], f"{name} whole n={n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_prompt_then_token_by_token(name, dtype, models):
    """A short prompt in one step, then ninety rows one at a time (long decoding through the cache and the state;
    steps of the same shape are replayed from a captured graph), and a sequence that is decoded from its first
    token on."""
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    ids = ids_for(name, 100, salt=1)
    st.step([("d", ids[:10])])
    for t in range(10, 100):
        st.step([("d", ids[t:t + 1])])
    close(st.rows("d", 100), plain_logits(models, name, ids), TOL[dtype], f"{name} decode")
    st.step([], end=["d"])
    ids = ids_for(name, 20, salt=2)
    for t in range(20):
        st.step([("e", ids[t:t + 1])])
    close(st.rows("e", 20), plain_logits(models, name, ids), TOL[dtype], f"{name} decode from the first token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
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
    close(st.rows("p", 131), plain_logits(models, name, ids), TOL[dtype], f"{name} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_unequal_requests_together_with_slots_and_pages_used_again(name, dtype, models):
    """Three state slots and 192 tokens of pages for six requests that need more in turn: portions of some beside
    single rows of others; a finished request's slot and pages go to the next one, whose state starts from zero.
    Every request's logits equal those of the request alone."""
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
        close(st.rows(r, n), plain_logits(models, name, ids[r]), TOL[dtype], f"{name} request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_a_row(dtype, models):
    """The same request whole, in portions and beside another request: float32 rows agree to rounding of sums
    (the products of a one-row step take another kernel), bfloat16 rows to bfloat16 rounding."""
    name = "P"
    ids = ids_for(name, 70, salt=9)
    other = ids_for(name, 40, salt=10)
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
        close(r, runs[0], 2e-5 if dtype == "float32" else 3e-2, "the same rows cut another way")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype, models):
    """The engine's own entry point, scheduler and sampling: greedy tokens follow the plain implementation's up
    to the first position where its two best logits are closer than the tolerance."""
    from nano_vllm_cpp_b200 import LLMEngine, SamplingParams
    name = "P"
    cfg, W, folder = models[name]
    prompts = [ids_for(name, 9, salt=20), ids_for(name, 3, salt=21), ids_for(name, 30, salt=22)]
    eng = LLMEngine(folder, max_model_len=96, num_kv_blocks=24, dtype=dtype, max_num_seqs=2, log_stats=False)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for k, tok in enumerate(o["token_ids"]):
            logits = pb.forward(cfg, W, seq)[-1]
            best = int(torch.argmax(logits))
            if best != tok:
                lead = float(logits[best] - logits[tok])
                bound = 2 * TOL[dtype] * float(logits.abs().max())
                assert lead <= bound, f"token {k} of a prompt of {len(p)}: {tok}, plain takes {best} with a lead of {lead:.3g}"
                break
            seq.append(tok)


def test_command_line_serves_the_design(models, tmp_path, capsys):
    """``nanovllm <folder> --tokens ...`` and ``nanovllm --config <json>`` (random weights) run this design as they
    run the other; the greedy tokens from the folder are the plain implementation's."""
    import json
    from nano_vllm_cpp_b200 import cli
    name = "Q"
    cfg, W, folder = models[name]
    prompt = ids_for(name, 7, salt=30)
    rc = cli.main([folder, "--tokens", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                   "--dtype", "float32", "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0, out
    toks = [int(t) for t in out.strip().splitlines()[-1].split(":")[1].split()]
    assert toks == pb.greedy_generate(cfg, W, prompt, 6)
    path = tmp_path / "config.json"
    path.write_text(json.dumps(CONFIGS["P"]))
    rc = cli.main(["--config", str(path), "--seed", "4", "--tokens", "5,6,7", "--max-tokens", "4", "--temperature", "0",
                   "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0 and len(out.strip().splitlines()[-1].split(":")[1].split()) == 4
