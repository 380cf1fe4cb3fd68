"""Mugulorn on the GPU against the plain implementation (tests/plain_mugulorn.py): every mechanism's kernels alone,
then whole models under every way of cutting the work, pages and state slots used again, long decoding, captured
steps, and greedy generation through the engine's entry point."""
import math

import numpy as np
import pytest
import torch

import plain_mugulorn as plain
import tiny_mugulorn as tm
import traces

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def _close(got, want, dtype, what, scale=None, f32=2e-5, bf16=2e-2):
    got, want = got.detach().double().cpu(), want.double()
    scale = float(want.abs().max()) if scale is None else scale
    tol = (f32 if dtype == "float32" else bf16) * max(scale, 1e-3)
    err = float((got - want).abs().max())
    assert math.isfinite(err) and err <= tol, f"{what}: max abs error {err:.3e} > {tol:.3e}"


def _rounded(t, dtype):
    """The values as a kernel gets them (inputs are stored in the activation type)."""
    return t.to(_dt(dtype)).double()


def _i32(x):
    return torch.as_tensor(x, dtype=torch.int32, device=DEV)


# ============================================================================= kernels alone


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dims,length,scaling", [(8, 8, tm._YARN), (16, 16, None), (4, 12, {"factor": 16.0, "original": 32, "fast": 4.0, "slow": 2.0}),
                                                 (64, 64, {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}), (0, 6, None)])
def test_rotation_by_stretched_frequencies(dims, length, scaling, dtype):
    """Pairs (i, i + dims/2) of the first ``dims`` numbers turn by position * frequency, what follows passes unchanged,
    at positions up to a hundred thousand; other columns of the destination are left alone."""
    from atom_b200 import native
    from atom_b200.parts.rope import RotaryYarn
    from atom_b200.parts.base import Runtime, Workspace

    pos_part = RotaryYarn(dims, 10000.0, scaling)
    rt = Runtime(_dt(dtype), torch.device(DEV), Workspace(torch.device(DEV)))
    g = torch.Generator().manual_seed(dims + length)
    T, n_vec, lead = 9, 3, 5
    x = _rounded(torch.randn(T, n_vec, lead + length, generator=g), dtype)
    positions = torch.tensor([0, 1, 2, 63, 64, 1000, 4097, 65536, 100001])
    out = torch.full((T, n_vec, 7 + length), 7.0, dtype=torch.float32, device=DEV)
    native.rotate_pairs(out, 7, x.to(_dt(dtype)).to(DEV), lead, length, dims, pos_part.frequencies(rt), pos_part.magnitude,
                        _i32(positions), _i32([0] * T))
    want = x[..., lead:].clone()
    if dims:
        freq, mag = plain.yarn_frequencies(dims, 10000.0, scaling)
        want[..., :dims] = plain.rotate_half(x[..., lead:lead + dims].transpose(0, 1), positions, freq, mag).transpose(0, 1)
    # angles are 32-bit: position * frequency carries a relative error of 2^-24, an absolute one that grows with the position
    out = out.cpu()
    _close(out[..., 7:], want, "float32", "rotated", f32=2e-2 if dims else 1e-7)
    near = positions < 5000
    _close(out[near][..., 7:], want[near], "float32", "rotated, near positions", f32=2e-3)
    assert bool((out[..., :7] == 7.0).all())


class LatentPages:
    """One request's latent rows laid into pages in a scrambled order, as the cache manager would."""

    def __init__(self, n_tokens, width, page, dtype, seed=0, extra_pages=5):
        g = torch.Generator().manual_seed(seed)
        n_pages = -(-n_tokens // page)
        order = torch.randperm(n_pages + extra_pages, generator=g)[:n_pages]
        self.table = order.to(torch.int32).view(1, -1).to(DEV)
        self.pages = torch.full((n_pages + extra_pages, page, width), float("nan"), dtype=dtype, device=DEV)
        self.page = page

    def fill(self, rows):
        for j in range(rows.shape[0]):
            self.pages[int(self.table[0, j // self.page]), j % self.page] = rows[j].to(self.pages.dtype)


def _plain_latent_scores(q, rows, R, scale, window, sink):
    """q [T, H, R + rd] folded queries, rows [T, R + rd]: the weighted sums of the rows' first R numbers."""
    T = q.shape[0]
    s = torch.einsum("ihd,jd->hij", q, rows) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & ((i - j < window) if window else True)
    s = s.masked_fill(~seen[None], -math.inf)
    if sink is None:
        a = torch.softmax(s, -1)
    else:
        top = torch.maximum(s.max(-1, keepdim=True).values, sink.view(-1, 1, 1))
        e = torch.exp(s - top)
        a = e / (e.sum(-1, keepdim=True) + torch.exp(sink.view(-1, 1, 1) - top))
    return torch.einsum("hij,jd->ihd", a, rows[:, :R])


def _run_latent(q, rows, R, rd, scale, window, sink, dtype, page, cuts, nsplit=0, kernel="plain"):
    from atom_b200 import native

    T, H, _ = q.shape
    dt = _dt(dtype)
    cache = LatentPages(T, R + rd, page, dt, seed=T)
    cache.fill(rows)
    out = torch.zeros(T, H, R, dtype=dt, device=DEV)
    sk = None if sink is None else sink.float().to(DEV)
    at = 0
    for n in cuts:
        n = min(n, T - at)
        if n <= 0:
            break
        ns = nsplit or native.attention_mixed_splits(n, min(at + n, window) if window else at + n)
        scratch = torch.empty(native.latent_attention_scratch_elems(n, H, R, ns), dtype=torch.float32, device=DEV) if ns > 1 else None
        o = torch.zeros(n, H, R, dtype=dt, device=DEV)
        if kernel.startswith("tc"):
            native.latent_attention_tc(o, q[at:at + n].float().contiguous().to(DEV), cache.pages, cache.table,
                                       _i32(range(at, at + n)), _i32([0, n]), 1, R, rd, scale, window, sk,
                                       ns, scratch, _i32([0] * n), rows=int(kernel[2:]))
        else:
            native.latent_attention(o, q[at:at + n].float().contiguous().to(DEV), cache.pages, cache.table,
                                    _i32(range(at, at + n)), _i32([0] * n), R, rd, scale, window, sk, ns, scratch)
        out[at:at + n] = o
        at += n
    assert at == T
    return out.double().cpu()


LATENT_CASES = [  # H, R, rd, window, page, T
    (4, 32, 8, 24, 16, 70), (2, 48, 16, 7, 8, 40), (3, 16, 4, 0, 8, 100), (5, 36, 12, 1, 16, 20), (1, 60, 20, 33, 16, 90),
    (8, 128, 32, 128, 32, 300), (16, 512, 64, 64, 64, 130), (7, 64, 32, 50, 16, 170), (3, 256, 0, 0, 16, 150),
    (70, 64, 32, 40, 8, 90), (5, 192, 32, 100, 16, 230), (2, 320, 16, 0, 32, 150),
]


def _kernels(H, R, rd, dtype):
    """The kernels that take these sizes: the plain one always, the tensor-core one (tiles of 64 and of 16 query rows) where
    it does."""
    from atom_b200 import native
    return ["plain", "tc64", "tc16"] if native.latent_attention_tc_supports(H, R, rd, _dt(dtype)) else ["plain"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", LATENT_CASES)
def test_latent_attention_in_prompts_portions_and_decoding(case, dtype):
    H, R, rd, window, page, T = case
    g = torch.Generator().manual_seed(H * R + T)
    q = torch.randn(T, H, R + rd, generator=g).double()
    rows = _rounded(torch.randn(T, R + rd, generator=g), dtype)
    sink = torch.randn(H, generator=g).double()
    scale = 2.0 / (R + rd) ** 0.5
    want = _plain_latent_scores(q.float().double(), rows, R, scale, window, sink)
    for kernel in _kernels(H, R, rd, dtype):
        for cuts in ([T], [T - 9] + [1] * 9, [13, 5, 2, 29, 2, 8, 3, 17] * 8):
            got = _run_latent(q, rows, R, rd, scale, window, sink, dtype, page, cuts, kernel=kernel)
            _close(got, want, dtype, f"{kernel}, cuts {cuts[:3]}", f32=2e-5, bf16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nsplit", [2, 3, 7, 40])
def test_latent_attention_with_keys_shared_out_among_blocks(nsplit, dtype):
    H, R, rd, window, page, T = 4, 64, 48, 0, 16, 333
    g = torch.Generator().manual_seed(nsplit)
    q = torch.randn(T, H, R + rd, generator=g).double()
    rows = _rounded(torch.randn(T, R + rd, generator=g), dtype)
    sink = torch.randn(H, generator=g).double()
    for kernel in _kernels(H, R, rd, dtype):
        for w in (0, 50):
            want = _plain_latent_scores(q.float().double(), rows, R, 0.3, w, sink)
            got = _run_latent(q, rows, R, rd, 0.3, w, sink, dtype, page, [T - 5, 1, 1, 1, 1, 1], nsplit=nsplit, kernel=kernel)
            _close(got, want, dtype, f"{kernel}, window {w}", f32=2e-5, bf16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 2, 16, 17, 40, 64, 300])
def test_one_key_at_the_windows_edge_stands_out(window, dtype):
    """One key row carries a mark that only it has and a score far above all others.  Queries at distance window - 1
    find the mark, queries at distance window do not: in a prompt, across portions that end at every place around
    the edge and a page's border, and decoded one by one."""
    H, R, rd, page, T = 2, 64, 32, 16, 420
    needle = 77
    g = torch.Generator().manual_seed(window)
    rows = torch.randn(T, R + rd, generator=g) * 0.1
    rows[:, 0] = 0.0
    rows[needle, 0] = 1.0                  # the mark, in the part that is summed
    rows[needle, R + 1] = 8.0              # ... and what the queries look for, in the part that is not
    rows = _rounded(rows, dtype)
    q = torch.randn(T, H, R + rd, generator=g).double() * 0.1
    q[:, :, 0] = 0.0
    q[:, :, R + 1] = 4.0
    sink = torch.tensor([-2.0, 0.5]).double()
    want = _plain_latent_scores(q.float().double(), rows, R, 1.0, window, sink)
    inside = [p for p in range(needle, T) if p - needle < window]
    outside = [p for p in range(needle + window, T)]
    assert all(want[p, :, 0].min() > 0.9 for p in inside) and all(want[p, :, 0].abs().max() == 0 for p in outside)
    edge = needle + window
    for cuts in ([T], [edge - 1, 1, 1, 1, T], [edge, T], [edge + 1, T], [needle + 1] + [1] * (T - needle - 1) if window <= 64 else [T],
                 [needle, 2, window, 2, T]):
        for kernel in _kernels(H, R, rd, dtype):
            if kernel == "tc64" and len(cuts) > 20:
                continue
            got = _run_latent(q, rows, R, rd, 1.0, window, sink, dtype, page, cuts, kernel=kernel)
            what = f"{kernel}, window {window}, cuts {cuts[:4]}"
            assert all(float(got[p, :, 0].min()) > 0.9 for p in inside), f"{what}: a key inside is lost"
            assert all(float(got[p, :, 0].abs().max()) == 0 for p in outside), f"{what}: a key outside is seen"
            _close(got, want, dtype, what, f32=2e-5, bf16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_counts_once_has_no_value_and_is_not_scaled(dtype):
    """With one key, the weight of its row is 1 / (1 + exp(sink - score)); a large sink empties the output."""
    H, R, rd = 3, 128, 16
    rows = _rounded(torch.ones(1, R + rd), dtype)
    q = torch.zeros(1, H, R + rd).double()
    q[:, :, 0] = torch.tensor([0.0, 1.0, -2.0]).double()
    sink = torch.tensor([0.0, 3.0, 40.0]).double()
    scale = 0.5
    want = 1.0 / (1.0 + torch.exp(sink - scale * q[0, :, 0]))
    for kernel in _kernels(H, R, rd, dtype):
        got = _run_latent(q, rows, R, rd, scale, 5, sink, dtype, 8, [1], kernel=kernel)
        _close(got[0, :, 0], want, dtype, f"sink, {kernel}", scale=1.0, f32=1e-6, bf16=4e-3)
    none = _run_latent(q, rows, R, rd, scale, 5, None, dtype, 8, [1])
    _close(none[0, :, 0], torch.ones(H).double(), dtype, "no sink", scale=1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,blocks,taps,lens", [
    (96, 3, 3, (37, 5, 18)), (128, 1, 2, (37, 5, 18)), (60, 5, 1, (37, 5, 18)), (140, 4, 8, (37, 5, 18)),
    (384, 4, 4, (37, 5, 18)), (80, 80, 4, (37, 5, 18)),
    (64, 2, 4, (300, 5, 40)), (48, 3, 12, (37, 5, 18)), (40, 2, 20, (290, 9, 4)), (72, 1, 7, (3, 530, 2))])
def test_convolution_and_recurrence_carry_over_steps(W, blocks, taps, lens, dtype):
    """Three requests of unequal lengths in one batch, fed whole, token by token and in portions down to two tokens,
    on state slots that held other requests before: the convolution's tail and the state go from step to step.  The
    long requests reach the kernels' forms for long steps (strips of rows, runs of a request side by side), the many
    taps the wider tap slots."""
    from atom_b200 import native

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(W + taps)
    bw = W // blocks
    lens = list(lens)
    P = {"y.b": torch.randn(W, generator=g) * 0.3, "x.b": torch.randn(W, generator=g) * 0.3,
         "conv": torch.randn(W, taps, generator=g) * 0.5, "conv.b": torch.randn(W, generator=g) * 0.2,
         "ra": torch.randn(blocks, bw, bw, generator=g) / bw ** 0.5, "ra.b": torch.randn(blocks, bw, generator=g),
         "ri": torch.randn(blocks, bw, bw, generator=g) / bw ** 0.5, "ri.b": torch.randn(blocks, bw, generator=g),
         "lam": torch.rand(W, generator=g) * 6.0 - 6.5}
    P = {k: _rounded(v, dtype) for k, v in P.items()}
    dev = {k: v.to(dt).to(DEV).contiguous() for k, v in P.items()}
    gates_w = torch.cat([dev["ra"], dev["ri"]], dim=1).contiguous()
    gates_b = torch.cat([dev["ra.b"], dev["ri.b"]], dim=1).contiguous()
    proj = [_rounded(torch.randn(n, 2 * W, generator=g), dtype) for n in lens]

    def reference(pr):
        """The mixer between its two products, by the plain functions (identity products around it)."""
        n = pr.shape[0]
        y = plain.gelu_tanh(pr[:, :W] + P["y.b"])
        u = plain.causal_conv(_rounded(pr[:, W:] + P["x.b"], dtype), P["conv"], P["conv.b"])
        u = _rounded(u, dtype)
        ub = u.view(n, blocks, bw)
        r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, P["ra"]) + P["ra.b"]).reshape(n, W)
        i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, P["ri"]) + P["ri.b"]).reshape(n, W)
        a = torch.exp(-8.0 * r * torch.nn.functional.softplus(P["lam"]))
        S, out = torch.zeros(W, dtype=F64), []
        for t in range(n):
            S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
            out.append(S * y[t])
        return torch.stack(out)

    want = [reference(p) for p in proj]
    n_slots = 5
    for cuts in ([1000], [1], [2], [7, 2, 3]) if max(lens) < 100 else ([1000], [270, 2, 1], [7, 280, 3]):
        state = torch.randn(n_slots, W, device=DEV)                       # what earlier requests left behind
        conv_state = torch.randn(n_slots, max(taps - 1, 1), W, device=DEV).to(dt)[:, :taps - 1].contiguous()
        slots = [3, 0, 4]
        for s in slots:                                                   # admission clears a request's slot
            state[s].zero_()
            conv_state[s].zero_()
        done = [0, 0, 0]
        got = [[] for _ in lens]
        k = 0
        while any(d < n for d, n in zip(done, lens)):
            live = [i for i in range(3) if done[i] < lens[i]]
            take = [min(cuts[(k + i) % len(cuts)], lens[i] - done[i]) for i in live]
            k += 1
            x = torch.cat([proj[i][done[i]:done[i] + n] for i, n in zip(live, take)]).to(dt).to(DEV).contiguous()
            T = x.shape[0]
            cu = _i32(np.concatenate([[0], np.cumsum(take)]))
            sot = _i32(np.repeat(np.arange(len(live)), take))
            ss = _i32([slots[i] for i in live])
            u = torch.empty(T, W, dtype=dt, device=DEV)
            native.causal_conv(u, x[:, W:], dev["x.b"], dev["conv"], dev["conv.b"], conv_state, sot, cu, ss)
            gates = torch.empty(T, blocks, 2 * bw, dtype=torch.float32, device=DEV)
            native.gemm_batched(gates, u.view(T, blocks, bw), gates_w)
            out = torch.empty(T, W, dtype=dt, device=DEV)
            native.rglru_scan(out, gates, gates_b, dev["lam"], u, x[:, :W], x[:, W:], dev["y.b"], dev["x.b"], state,
                              conv_state, cu, ss, len(live), taps, 8.0, True)
            at = 0
            for i, n in zip(live, take):
                got[i].append(out[at:at + n].double().cpu())
                at += n
                done[i] += n
        for i in range(3):
            _close(torch.cat(got[i]), want[i], dtype, f"cuts {cuts}, request {i}", f32=3e-5, bf16=3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_state_remembers_a_token_hundreds_of_steps_back(dtype):
    """A channel whose decay is nearly one keeps a single early input through 600 single-token steps; a channel that
    decays fast has forgotten it.  (sqrt(1 - a^2) near a = 1 is where a careless form loses the input.)"""
    from atom_b200 import native

    dt = _dt(dtype)
    W, taps, n = 64, 1, 600
    lam = torch.full((W,), -9.0)
    lam[W // 2:] = 2.0
    zeros = torch.zeros(W, dtype=dt, device=DEV)
    conv_w = torch.ones(W, 1, dtype=dt, device=DEV)
    gates_b = torch.zeros(1, 2 * W, dtype=dt, device=DEV)
    state = torch.zeros(1, W, device=DEV)
    conv_state = torch.zeros(1, 0, W, dtype=dt, device=DEV)
    outs = []
    for t in range(n):
        x = torch.zeros(1, 2 * W, dtype=dt, device=DEV)
        x[:, :W] = 3.0                      # y: gelu(3) ~ 2.99
        if t == 2:
            x[:, W:] = 1.0
        u = torch.empty(1, W, dtype=dt, device=DEV)
        native.causal_conv(u, x[:, W:], zeros, conv_w, zeros, conv_state, _i32([0]), _i32([0, 1]), _i32([0]))
        gates = torch.zeros(1, 1, 2 * W, dtype=torch.float32, device=DEV)          # r = i = 1/2
        out = torch.empty(1, W, dtype=dt, device=DEV)
        native.rglru_scan(out, gates, gates_b, lam.to(dt).to(DEV), u, x[:, :W], x[:, W:], zeros, zeros, state, conv_state,
                          _i32([0, 1]), _i32([0]), 1, taps, 8.0, True)
        outs.append(out[0].double().cpu())
    lam64 = _rounded(lam, dtype)
    a = torch.exp(-8.0 * 0.5 * torch.nn.functional.softplus(lam64))
    want = a ** (n - 3) * torch.sqrt(1 - a * a) * 0.5 * float(plain.gelu_tanh(torch.tensor(3.0, dtype=F64)))
    assert float(want[0]) > 0.005 and float(want[-1]) == 0.0
    _close(outs[-1], want, dtype, "after 600 steps", f32=1e-4, bf16=1e-2)
    assert float(outs[1].abs().max()) == 0.0            # nothing before the input


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_kernels(dtype):
    """gelu-gated product, sigmoid gate over rows that lie apart, residual add times a constant, batched products."""
    from atom_b200 import native

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(1)
    for n in (52, 72):        # 72: the form with 16-byte loads
        gu = _rounded(torch.randn(7, 2 * n, generator=g) * 3, dtype)
        out = torch.empty(7, n, dtype=dt, device=DEV)
        native.gelu_mul(out, gu.to(dt).to(DEV))
        _close(out, plain.gelu_tanh(gu[:, :n]) * gu[:, n:], dtype, f"gelu_mul {n}")

    for width, at, n in ((100, 70, 30), (104, 64, 40)):       # the second: the form with 16-byte loads
        wide = _rounded(torch.randn(5, width, generator=g) * 3, dtype)
        x = _rounded(torch.randn(5, n, generator=g), dtype)
        xd = x.to(dt).to(DEV).contiguous()
        native.sigmoid_mul(xd, wide.to(dt).to(DEV)[:, at:])
        _close(xd, x * torch.sigmoid(wide[:, at:]), dtype, f"sigmoid_mul {n}")

    res = torch.randn(6, 100, generator=g)
    delta = _rounded(torch.randn(6, 100, generator=g), dtype)
    w = _rounded(torch.rand(100, generator=g) + 0.5, dtype)
    rd = res.to(DEV).contiguous()
    o = torch.empty(6, 100, dtype=dt, device=DEV)
    native.add_rmsnorm(o, rd, delta.to(dt).to(DEV), w.to(dt).to(DEV), 1e-5, delta_scale=0.3)
    r = res.double() + 0.3 * delta
    _close(rd, r, "float32", "residual + 0.3 delta", f32=1e-6)
    _close(o, plain.rms_norm(r, w, 1e-5), dtype, "norm of it")

    a = _rounded(torch.randn(9, 3, 20 + 4, generator=g), dtype)
    wt = _rounded(torch.randn(3, 11, 20, generator=g), dtype)
    ad = a.to(dt).to(DEV)
    for out_dt in ([torch.float32] if dtype == "float32" else [torch.float32, torch.bfloat16]):
        full = torch.zeros(9, 3, 11 + 2, dtype=out_dt, device=DEV)
        native.gemm_batched(full[:, :, :11], ad[:, :, :20], wt.to(dt).to(DEV).contiguous())
        _close(full[:, :, :11], torch.einsum("mbk,bnk->mbn", a[:, :, :20], wt), "float32" if out_dt == torch.float32 else dtype, "batched")
        assert bool((full[:, :, 11:] == 0).all())


# ============================================================================= whole models

LENGTHS = {"A": [1, 2, 9, 41, 100, 70], "B": [3, 17, 64, 131, 30], "C": [5, 33, 90, 48, 70], "D": [4, 70, 150, 33]}
TOL = {"float32": 2e-4, "bfloat16": 8e-2}
RMS_TOL_BF16 = 1.5e-2


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for name, cfg in tm.CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"mugulorn_{name}"))
        tm.write_model(cfg, d, tm.SEEDS[name])
        out[name] = d
    return out


_plain_memo = {}


def _plain_logits(model_dir, seqs):
    if model_dir not in _plain_memo:
        _plain_memo[model_dir] = tm.read_model(model_dir) + ({},)
    cfg, w, memo = _plain_memo[model_dir]
    out = {}
    for rid, toks in seqs.items():
        key = tuple(toks)
        if key not in memo:
            memo[key] = plain.forward(cfg, w, list(toks)).numpy()
        out[rid] = memo[key]
    return out


def _runner(model_dir, dtype, max_tokens, page, max_num_seqs=4, **kw):
    from atom_b200.config import EngineConfig
    from atom_b200.engine.runner import ModelRunner

    kw.setdefault("enforce_eager", True)
    return ModelRunner(EngineConfig(model=model_dir, dtype=dtype, kv_cache_block_size=page,
                                    num_kvcache_blocks=max(1, -(-max_tokens // page)), max_num_seqs=max_num_seqs, **kw))


def _replay(runner, steps):
    from atom_b200.engine.batch import StepEntry

    out = {}
    for s in steps:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in s["entries"]])
        runner.check_status()
        if logits.shape[0]:
            out[s["step"]] = logits.float().cpu().numpy()
        for rid in s.get("end", []):
            runner.finish(rid)
        runner.cache.check()
    return out


def _compare(got, ref, dtype, what):
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = TOL[dtype] * max(1.0, scale)
    for rid, r in ref.items():
        g = got[rid]
        assert g.shape == r.shape and np.isfinite(g).all(), f"{what}: {rid}"
        e = np.abs(g.astype(np.float64) - r).max(axis=1)
        assert e.max() <= tol, f"{what}: {rid}[{int(e.argmax())}] off by {e.max():.3e} > {tol:.3e}"
        if dtype == "bfloat16":
            rms = float(np.sqrt(((g - r) ** 2).mean()))
            assert rms <= RMS_TOL_BF16 * scale, f"{what}: rms error {rms:.3e} in {rid}"
        else:
            assert (g.argmax(1) == r.argmax(1)).all(), f"{what}: greedy token differs in {rid}"


def _seqs(name):
    ps = tm.prompts(tm.CONFIGS[name], LENGTHS[name], seed=len(name) + ord(name))
    return {f"r{i}": p for i, p in enumerate(ps)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_by_layer_against_plain(dirs, dtype):
    """The residual stream after every layer of a short prompt (what the next norm reads)."""
    from atom_b200.engine.batch import StepEntry
    name = "A"
    cfg, w = tm.read_model(dirs[name])
    p = tm.prompts(tm.CONFIGS[name], [29], seed=2)[0]
    want = []
    plain.forward(cfg, w, p, want)
    runner = _runner(dirs[name], dtype, 64, tm.PAGE[name])
    seen = []
    for b in runner.model.blocks:
        def run(residual, delta, step, cache, wc, delta_scale=None, _o=b.run, _b=b):
            out = _o(residual, delta, step, cache, wc, delta_scale=delta_scale)
            seen.append(residual.double() + _b.delta_scale * out.double())
            return out
        b.run = run
    runner.step([StepEntry("a", p, [0])])
    runner.check_status()
    assert len(seen) == len(want)
    for i, (g, r) in enumerate(zip(seen, want)):
        _close(g, r, dtype, f"after layer {i}", f32=2e-5, bf16=2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tm.CONFIGS))
def test_every_cut_matches_plain(dirs, name, dtype):
    """Whole; the last 48 tokens one by one (every window of these models passes over decoded tokens); portions of
    changing size down to two tokens; pairs of tokens throughout; up to four live requests with portions beside single
    tokens in a pool so small that pages and state slots are used again."""
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    mixed, peak = traces.mixed(seqs, max_live=4, budget_tokens=320)
    assert peak <= 320 < sum(-(-len(t) // 64) * 64 for t in seqs.values())
    runner = _runner(dirs[name], dtype, 320, tm.PAGE[name], max_num_seqs=4)
    for what, steps in (("whole", traces.whole(seqs)), ("tail", traces.tail_by_token(seqs, 48)),
                        ("ragged", traces.ragged(seqs)), ("pairs", traces.ragged(seqs, sizes=(2,))), ("mixed", mixed)):
        if what == "pairs":
            steps = [s for s in steps if s["entries"][0]["id"] in ("r1", "r2")]       # (two short requests are enough)
            sub = {r: ref[r] for r in ("r1", "r2")}
            _compare(traces.collect(steps, _replay(runner, steps)), sub, dtype, f"{name}/{what}")
            continue
        _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, f"{name}/{what}")
        assert all(g.pool.num_used == 0 for g in runner.cache.groups) and runner.cache.state_slots.num_free == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_request_freed_half_way_and_fed_again(dirs, name, dtype):
    """What preemption by recomputation does: pages and the state slot go back, another request takes them, and the
    victim starts over on whatever slot is free, with a state of zeros."""
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    ids = list(seqs)
    steps, peak = traces.mixed_refeed(seqs, [ids[-1], ids[-2]], max_live=3, budget_tokens=384)
    runner = _runner(dirs[name], dtype, peak, tm.PAGE[name], max_num_seqs=3)
    rows = traces.collect_rows(steps, _replay(runner, steps))
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = TOL[dtype] * max(1.0, scale)
    for rid, got in rows.items():
        assert {p for p, _ in got} == set(range(len(seqs[rid])))
        errs = [float(np.abs(row.astype(np.float64) - ref[rid][p]).max()) for p, row in got]
        assert max(errs) <= tol, f"{name}/{dtype}: {rid}: worst {max(errs):.3e} > {tol:.3e}"
    assert all(g.pool.num_used == 0 for g in runner.cache.groups) and runner.cache.state_slots.num_free == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_of_unequal_requests_equals_each_alone(dirs, dtype):
    """The same rows, computed alone and beside three other requests of other lengths, differ by rounding at most."""
    name = "B"
    ps = tm.prompts(tm.CONFIGS[name], [50, 3, 27, 64], seed=99)
    runner = _runner(dirs[name], dtype, 1024, tm.PAGE[name])
    from atom_b200.engine.batch import StepEntry
    alone = []
    for i, p in enumerate(ps):
        alone.append(runner.step([StepEntry(("a", i), p, list(range(len(p))))]).float().cpu().numpy())
        runner.finish(("a", i))
    both = runner.step([StepEntry(("b", i), p, list(range(len(p)))) for i, p in enumerate(ps)]).float().cpu().numpy()
    at = 0
    for i, p in enumerate(ps):
        part = both[at:at + len(p)]
        at += len(p)
        scale = float(np.abs(alone[i]).max())
        assert np.abs(part - alone[i]).max() <= (1e-4 if dtype == "float32" else 4e-2) * scale
    runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_token_by_token(dirs, dtype):
    """300 tokens decoded one by one after a prompt of three: pages fill, follow one another and are given back as
    the windows pass; the state and the convolution's tail are read and written 300 times."""
    name = "A"
    p = tm.prompts(tm.CONFIGS[name], [303], seed=4)[0]
    seqs = {"long": p}
    ref = _plain_logits(dirs[name], seqs)
    steps = traces.tail_by_token(seqs, 300)
    runner = _runner(dirs[name], dtype, 96, tm.PAGE[name])          # (a pool that only the window's pages fit into)
    _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_match_plain(dirs, dtype):
    """Decode steps and small mixed steps replayed from CUDA graphs, with padding rows and padding requests."""
    name = "B"
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    runner = _runner(dirs[name], dtype, 1024, tm.PAGE[name], max_num_seqs=8, enforce_eager=False,
                     cudagraph_capture_sizes=[1, 2, 4], max_model_len=256)
    for what, steps in (("tail", traces.tail_by_token(seqs, 32)), ("mixed", traces.mixed(seqs, max_live=3, tail=40)[0]),
                        ("ragged", traces.ragged(seqs))):
        _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, f"graphs/{what}")
    assert runner.graph_replays > 50
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


def _plain_greedy(cfg, w, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(plain.forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("name,chunk", [("A", 8), ("C", 13)])
def test_greedy_generation_through_the_engine_fp32(dirs, name, chunk):
    from atom_b200 import LLMEngine, SamplingParams
    cfg, w = tm.read_model(dirs[name])
    prompts = tm.prompts(tm.CONFIGS[name], [1, 7, 16, 33], seed=21)
    eng = LLMEngine(dirs[name], dtype="float32", kv_cache_block_size=tm.PAGE[name], num_kvcache_blocks=64,
                    enforce_eager=(name == "C"), max_num_batched_tokens=chunk + 4, long_prefill_token_threshold=chunk,
                    max_num_seqs=4)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o["num_tokens_output"] == 10
        assert o["token_ids"] == _plain_greedy(cfg, w, p, 10)
    assert all(g.pool.num_used == 0 for g in eng.runner.cache.groups)


def test_greedy_generation_bf16_with_preemption(dirs):
    """A pool so small that requests are preempted and computed again; every token stays within rounding of the
    plain implementation's best."""
    from atom_b200 import LLMEngine, SamplingParams
    name = "B"          # (its third layer keeps every row, so pages do run out)
    cfg, w = tm.read_model(dirs[name])
    prompts = tm.prompts(tm.CONFIGS[name], [3, 5, 12, 29], seed=5)
    eng = LLMEngine(dirs[name], dtype="bfloat16", kv_cache_block_size=8, num_kvcache_blocks=14, max_num_batched_tokens=24,
                    max_num_seqs=4, enforce_eager=True)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    assert eng.stats()["preemptions"] > 0
    for p, o in zip(prompts, outs):
        full = list(p) + o["token_ids"]
        logits = plain.forward(cfg, w, full[:-1]).numpy()
        for i, tok in enumerate(o["token_ids"]):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 0.15, f"token {i}: logit {row[tok]:.3f} against {row.max():.3f}"
    eng.runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_on_a_mugulorn_folder(dirs, tmp_path, dtype):
    """bin/trace_run as a user runs it (a child process, steps on standard input, one file of logits per step): the
    model class is chosen by config.json; four state slots and a pool smaller than the requests' sum."""
    import json
    import os
    import subprocess
    import sys

    name = "A"
    seqs = _seqs(name)
    steps, peak = traces.mixed(seqs, max_live=4, budget_tokens=320)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / f"out_{dtype}"
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dirs[name], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(peak)], input=text, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(l.split()[1]) for l in p.stdout.splitlines() if l.startswith("done ")] == [s["step"] for s in steps]
    V = tm.CONFIGS[name]["vocab"]
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        if n:
            a = np.fromfile(out / f"{s['step']}.f32", dtype="<f4")
            assert a.size == n * V
            outputs[s["step"]] = a.reshape(n, V)
    _compare(traces.collect(steps, outputs), _plain_logits(dirs[name], seqs), dtype, f"trace_run/{dtype}")
