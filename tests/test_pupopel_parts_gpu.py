"""Every mechanism of Pupopel alone on the GPU against the plain functions, at sizes of its own: the gated delta rule with a
decay per key channel through its state slots (token by token and in chunks), softmax attention with normed queries and
keys, a query factor by position, a bias by distance and a sink through its pages, lightning attention, the pair of
mixers, the router over raw outputs with a bias and a shared expert, the dense gated layer, the block whose sublayers read
one norm, and the product that opens a pass of the loop.  Requests run in portions of many sizes beside one another;
slots and pages are freed and used again (freed memory is NaN)."""
import math

import pytest
import torch

from plain import pupopel_plain as P
from test_parts_gpu import cache_for, give_weights, runtime, step_in_portions

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}
CUTS = [[37, 0, 9], [5, 20, 1], [1, 1, 1], [2, 3, 1], [64, 2, 1], [1, 30, 2], [200, 200, 200]]
LENGTHS = [130, 61, 40]
WIDTH = 56


def close(got, want, dtype, tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= (tol or TOL[dtype]), f"error {err:.3g}"


def inputs(lengths, width, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(dtype) for n in lengths]


def rows_of(xs, spans):
    return torch.cat([xs[r][lo:hi] for r, lo, hi in spans]).cuda()


def f64(stored):
    return {k: v.double() for k, v in stored.items()}


def rebind(part, stored, dtype):
    from logssms_b200.weights.loader import check_and_place
    part.bind_tree(check_and_place(part, {k: v.to(dtype) for k, v in stored.items()}, dtype, "cuda"))


# --------------------------------------------------------------------------- gated delta rule
def delta_part(dtype, heads, kv_heads, dim, vdim, conv, rank_a=6, rank_g=5, seed=0, eps=1e-5):
    from logssms_b200.config.specs import DeltaRuleSpec
    from logssms_b200.parts import ChannelDelta
    spec = DeltaRuleSpec(WIDTH, heads, kv_heads, dim, vdim, conv, eps, decay_rank=rank_a, gate_rank=rank_g)
    part = ChannelDelta(spec, perturb_init=True)
    stored = give_weights(part, dtype, seed=seed)
    return part, stored, dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, eps=eps)


def plain_delta(x, stored, kw):
    return P.channel_delta(x.double(), f64(stored), {}, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, conv", [
    (4, 2, 16, 24, 3), (2, 2, 32, 16, 4), (3, 3, 8, 136, 1), (6, 1, 24, 8, 2), (1, 1, 2, 1, 2), (2, 1, 40, 72, 4),
    (3, 1, 12, 5, 5), (2, 2, 72, 12, 8), (4, 4, 64, 32, 4), (2, 1, 136, 40, 3)])
def test_delta_rule_in_portions(dtype, heads, kv_heads, dim, vdim, conv):
    if vdim == 1 and dtype == torch.bfloat16:
        # a norm over one channel is x / sqrt(x^2 + eps), the sign of x unless x is tiny: bfloat16's rounding of a small x
        # moves it by more than any tolerance; the float32 run covers the sizes of 1
        pytest.skip("a norm over one channel is a sign")
    part, stored, kw = delta_part(dtype, heads, kv_heads, dim, vdim, conv, seed=heads + dim)
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3)
    xs = inputs(LENGTHS, WIDTH, dtype, seed=1)
    for _ in range(2):                            # twice: the second time through slots that were freed (and hold NaN)
        got = step_in_portions(planner, cache, LENGTHS, CUTS, lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, plain_delta(x, stored, kw), dtype)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, conv", [(4, 2, 64, 32, 4), (2, 2, 16, 40, 2), (3, 1, 128, 128, 4), (2, 2, 48, 24, 3),
                                                              (1, 1, 256, 16, 4), (1, 1, 300, 6, 2), (2, 1, 17, 3, 3)])
def test_delta_rule_of_long_portions_carries_the_state_from_chunk_to_chunk_and_step_to_step(heads, kv_heads, dim, vdim, conv):
    """Portions of hundreds of tokens (the kernel of long portions, whose rows arrive sixteen or eight tokens at a time)
    beside a short request and single tokens (the token-by-token kernel), cut inside those blocks."""
    for dtype in DTYPES:
        part, stored, kw = delta_part(dtype, heads, kv_heads, dim, vdim, conv, seed=dim)
        cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3, max_seq_len=1024)
        lengths = [700, 9, 420]
        xs = inputs(lengths, WIDTH, dtype, seed=2)
        got = step_in_portions(planner, cache, lengths, [[301, 2, 0], [250, 1, 420], [1, 1, 0], [148, 5, 0]],
                               lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, plain_delta(x, stored, kw), dtype)


def test_delta_rule_remembers_a_token_hundreds_of_steps_back():
    """Decays next to 1 and one early token whose input is by far the largest: what it wrote is still read 600 tokens
    later, through prompts, portions of two tokens and single tokens."""
    dtype = torch.float32
    part, stored, kw = delta_part(dtype, 2, 1, 16, 8, 3, seed=4)
    stored["A_log"] = torch.full_like(stored["A_log"], -9.0)
    rebind(part, stored, dtype)
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=2, max_seq_len=1024)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(640, WIDTH, generator=g) * 0.2
    x[5] *= 30.0
    cuts = [[300], [1], [1], [2], [250]] + [[1]] * 86
    (got,) = step_in_portions(planner, cache, [640], cuts, lambda ctx, spans: part.forward(rows_of([x], spans), ctx, 0))
    want = plain_delta(x, stored, kw)
    close(got, want, dtype)
    blind = x.clone()
    blind[5] = 0.0
    other = plain_delta(blind, stored, kw)
    assert float((want - other)[-50:].abs().max() / want[-50:].abs().max()) > 0.05


def test_delta_rule_overwrites_what_a_key_held():
    """The rule itself, on the kernel alone: with a write gate of 1, no decay and the same unit key twice, the second value
    replaces the first one (a plain sum of outer products would read back their sum)."""
    from logssms_b200.ops import kernels as K
    dim, vdim = 8, 4
    T = 3
    qkv = torch.zeros(T, 2 * dim + vdim)
    key = torch.zeros(dim)
    key[2] = 5.0                                   # its unit vector is e_2 (up to the 1e-6 inside the root)
    qkv[:, :dim] = key                             # queries = keys
    qkv[:, dim:2 * dim] = key
    qkv[0, 2 * dim:] = torch.tensor([1.0, 2.0, 3.0, 4.0])
    qkv[1, 2 * dim:] = torch.tensor([-1.0, 0.5, 0.0, 9.0])
    qkv[2, 2 * dim:] = qkv[1, 2 * dim:]
    z = torch.full((T, dim), -40.0)                # softplus(-40) = 0: the decay is 1
    beta = torch.full((T, 1), 40.0)                # sigmoid(40) = 1
    state = torch.full((1, 1, dim, vdim), float("nan"))
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32).cuda()
    o = K.delta_scan(qkv.cuda(), z.cuda(), torch.zeros(dim).cuda(), torch.zeros(1).cuda(), beta.cuda(), state.cuda(), i32(0, T), i32(0),
                     i32(0), 1, 1, 1, dim, vdim, 1.0, 1e-6)
    assert torch.allclose(o.cpu(), qkv[:, 2 * dim:], atol=1e-5)


def slow_delta_recurrence(q, k, v, z, dt, A, beta, S, heads, kv_heads, dim, vdim):
    """The recurrence token by token in float64, from its equations: q, k [T, kv_heads * dim], v [T, heads * vdim],
    z [T, heads * dim], beta [T, heads]; S [heads, dim, vdim] is updated in place."""
    T = q.shape[0]
    o = torch.zeros(T, heads, vdim, dtype=torch.float64)
    for t in range(T):
        for h in range(heads):
            hk = h // (heads // kv_heads)
            qt, kt = q[t, hk * dim:(hk + 1) * dim], k[t, hk * dim:(hk + 1) * dim]
            qt = qt / torch.sqrt((qt * qt).sum() + 1e-6) * dim ** -0.5
            kt = kt / torch.sqrt((kt * kt).sum() + 1e-6)
            g = torch.exp(-torch.exp(A[h]) * torch.nn.functional.softplus(z[t, h * dim:(h + 1) * dim] + dt[h * dim:(h + 1) * dim]))
            S[h] = g[:, None] * S[h]
            u = torch.sigmoid(beta[t, h]) * (v[t, h * vdim:(h + 1) * vdim] - S[h].T @ kt)
            S[h] = S[h] + kt[:, None] * u[None, :]
            o[t, h] = S[h].T @ qt
    return o.reshape(T, heads * vdim)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(2, 1, 5, 3), (3, 3, 24, 40), (2, 2, 64, 33), (4, 2, 100, 16), (1, 1, 128, 130), (1, 1, 200, 9), (2, 1, 300, 8)])
@pytest.mark.parametrize("kernel", ["delta_scan", "delta_scan_rows", "delta_scan_chunks"])
def test_delta_rule_kernels_equal_the_recurrence_written_out(kernel, heads, kv_heads, dim, vdim):
    """The three kernels alone: two portions side by side whose lengths are no multiples of anything, the second going on
    from a state it is handed in another slot; decays from none to a thousandfold per token (a chunk's running decay
    underflows in some channels, so only differences of log-decays may ever be exponentiated)."""
    from logssms_b200.ops import kernels as K
    from logssms_b200.parts.context import chunk_lists
    if kernel == "delta_scan_chunks" and not K.delta_scan_chunks_ok(dim):
        pytest.skip("more key channels than the chunked kernel takes")
    g = torch.Generator().manual_seed(dim + vdim)
    lens = [37, 8 * 9 + 3]
    T = sum(lens)
    q = torch.randn(T, kv_heads * dim, generator=g, dtype=torch.float64)
    k = torch.randn(T, kv_heads * dim, generator=g, dtype=torch.float64)
    v = torch.randn(T, heads * vdim, generator=g, dtype=torch.float64)
    z = torch.randn(T, heads * dim, generator=g, dtype=torch.float64) * 3.0
    z[:, ::3] += 6.0                                # strong decays in every third channel ...
    z[:, 1::3] -= 30.0                              # ... and none at all in the next
    dt = torch.randn(heads * dim, generator=g, dtype=torch.float64)
    A = torch.rand(heads, generator=g, dtype=torch.float64) * 2.0 - 1.5
    beta = torch.randn(T, heads, generator=g, dtype=torch.float64) * 2.0
    handed = torch.randn(heads, dim, vdim, generator=g, dtype=torch.float64)
    want, states = [], []
    for r, (lo, n) in enumerate(((0, lens[0]), (lens[0], lens[1]))):
        S = torch.zeros(heads, dim, vdim, dtype=torch.float64) if r == 0 else handed.clone()
        want.append(slow_delta_recurrence(q[lo:lo + n], k[lo:lo + n], v[lo:lo + n], z[lo:lo + n], dt, A, beta[lo:lo + n], S,
                                          heads, kv_heads, dim, vdim))
        states.append(S)
    want = torch.cat(want)
    i32 = lambda *x: torch.tensor(x, dtype=torch.int32).cuda()
    state = torch.full((3, heads, dim, vdim), float("nan"))
    state[2] = handed.float()                       # request 1 lives in slot 2; request 0 starts at position 0 in slot 0 (NaN there)
    state = state.cuda()
    qkv = torch.cat([q, k, v], 1).float().cuda()
    common = (qkv, z.float().cuda(), dt.float().cuda(), A.float().cuda(), beta.float().cuda(), state, i32(0, lens[0], T), i32(0, 500), i32(0, 2))
    sizes = (heads, kv_heads, dim, vdim, dim ** -0.5, 1e-6)
    if kernel == "delta_scan_chunks":
        chunks, per_request = chunk_lists(lens, K.DELTA_CHUNK)
        o = K.delta_scan_chunks(*common, torch.from_numpy(chunks).cuda(), chunks.shape[0], torch.from_numpy(per_request).cuda(),
                                per_request.shape[0], *sizes)
    else:
        o = getattr(K, kernel)(*common, 2, *sizes)
    close(o, want, torch.float32, 2e-5)
    close(state[0], states[0], torch.float32, 2e-5)
    close(state[2], states[1], torch.float32, 2e-5)
    assert torch.isnan(state[1]).all()
