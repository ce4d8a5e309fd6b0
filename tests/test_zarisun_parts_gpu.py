"""Every mechanism of Zarisun alone on the GPU against the plain functions, at sizes of its own: windowed attention over
convolved keys with whole-row norms, neighbour rotation with stretched frequencies, a sink and a gate per head; attention over
cached latents with a sink and a gate, also from another layer's cache; the gated delta rule with one decay per head; the
block whose norms sit on the sublayers' outputs; and the small kernels they added.  Requests run in portions of many sizes
beside one another; slots and pages are freed and used again (freed memory is NaN)."""
import math

import pytest
import torch

from plain import zarisun_plain as P
from test_parts_gpu import cache_for, give_weights, runtime, step_in_portions

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}
CUTS = [[37, 0, 9], [5, 20, 1], [1, 1, 1], [2, 3, 1], [64, 2, 1], [1, 30, 2], [200, 200, 200]]
LENGTHS = [130, 61, 40]
WIDTH = 56
EPS = 1e-5


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


def rope_spec(part_dim, rot):
    from logssms_b200.config.specs import RopeSpec
    if rot is None:
        return None
    sc = rot.get("scaling")
    return RopeSpec(part_dim, rot["dims"], rot["base"], 4096, None if sc is None else tuple(sorted((k, float(v)) for k, v in sc.items())),
                    kind="rope_ramp")


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


# --------------------------------------------------------------------------- the rotation table
@pytest.mark.parametrize("r", [rot(8, 16.0), rot(8, 16.0, (4.0, 64, 4.0, 1.0)), rot(32, 40000.0, (4.0, 1024, 16.0, 2.0)), rot(2, 7.0, (3.0, 8, 2.0, 1.0))])
def test_rotation_table(r):
    from logssms_b200.parts.rope import RampRotaryEmbedding
    enc = RampRotaryEmbedding(rope_spec(r["dims"], r))
    enc.setup(runtime(torch.float32, max_seq_len=700))
    f, mag = P.yarn_frequencies(r)
    a = torch.arange(700, dtype=torch.float64)[:, None] * f.float().double()[None, :]       # the engine's frequencies are float32
    want = torch.cat([torch.cos(a), torch.sin(a)], 1) * mag
    assert enc.table.shape == (700, r["dims"])
    assert float((enc.table.double().cpu() - want).abs().max()) < 1e-4        # float32 angles of up to 700 radians


# --------------------------------------------------------------------------- windowed attention over convolved keys
def attention_part(dtype, heads, kv_heads, dim, conv, window, r, scale=0.3, seed=0, max_seq_len=256):
    from logssms_b200.config.specs import ConvAttentionSpec
    from logssms_b200.parts import ConvAttention
    spec = ConvAttentionSpec(WIDTH, heads, kv_heads, dim, conv, scale, window, rope_spec(dim, r), EPS)
    part = ConvAttention(spec, perturb_init=True)
    stored = give_weights(part, dtype, seed=seed)
    part.setup(runtime(dtype, max_seq_len=max_seq_len))
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "conv": conv, "scale": scale, "rot": r,
         "mask": None if window is None else {"size": window}}
    return part, stored, m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, conv, window, r", [
    (6, 2, 16, 3, 20, rot(8, 500.0, (8.0, 32, 16.0, 2.0))), (4, 1, 32, 2, 70, rot(32, 10000.0)), (2, 2, 16, 1, 1, None),
    (1, 1, 2, 1, 2, rot(2, 100.0)), (4, 2, 8, 4, 64, rot(4, 1000.0)), (2, 1, 24, 5, None, rot(24, 8000.0, (16.0, 128, 32.0, 1.0))),
    (3, 3, 40, 8, 17, rot(6, 30.0, (2.0, 8, 4.0, 0.5))), (8, 2, 64, 4, 33, rot(16, 30000.0, (4.0, 256, 16.0, 1.0))), (5, 1, 6, 3, 16, rot(6, 9.0))])
def test_conv_attention_in_portions(dtype, heads, kv_heads, dim, conv, window, r):
    part, stored, m = attention_part(dtype, heads, kv_heads, dim, conv, window, r, seed=heads + dim)
    # sharp queries: single keys carry the output, so one that is missing or surplus shows
    stored["q.norm"] = stored["q.norm"] * (4.0 if dtype == torch.float32 else 1.5)
    rebind(part, stored, dtype)
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3)
    xs = inputs(LENGTHS, WIDTH, dtype, seed=1)
    for _ in range(2):                            # twice: the second time through slots and pages that were freed (and hold NaN)
        got = step_in_portions(planner, cache, LENGTHS, CUTS, lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, P.conv_attention(x.double(), f64(stored), m, EPS), dtype)


@pytest.mark.parametrize("window", [1, 2, 5, 16, 17, 31, 64, 65])
@pytest.mark.parametrize("cuts", [[[200]], [[3], [2], [40], [2], [200]], [[50]] + [[1]] * 110, [[1]] * 40 + [[29], [200]]])
def test_window_names_its_keys(window, cuts):
    """Queries of zero make all scores equal: the output is then sum of the window's values / (count + exp(sink)).  The values
    (the convolved keys) carry a one and the token's position, so every output names how many keys were seen and which: in
    prompts cut anywhere, in decoded tokens, over pages of 16."""
    dtype = torch.float32
    n, dim = 160, 4
    part, stored, m = attention_part(dtype, 1, 1, dim, 3, window, None, seed=3)
    stored["q"] = torch.zeros_like(stored["q"])
    stored["k"] = torch.zeros_like(stored["k"])
    stored["k"][0, 0] = 1.0                                  # key channel 0 = input column 0 (a one), channel 1 = column 1 (the position)
    stored["k"][1, 1] = 1.0
    stored["k.conv"] = torch.tensor([[0.0, 0.0, 1.0]]).repeat(dim, 1)         # the current token's tap alone
    stored["g"] = torch.zeros_like(stored["g"])              # gate: sigmoid(0) = 1/2
    stored["sink"] = torch.tensor([math.log(3.0)])
    stored["o"] = torch.zeros_like(stored["o"])
    stored["o"][0, 0] = 1.0
    stored["o"][1, 1] = 1.0
    rebind(part, stored, dtype)
    x = torch.zeros(n, WIDTH)
    x[:, 0] = 1.0
    x[:, 1] = torch.arange(n, dtype=torch.float32)
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=2)
    (got,) = step_in_portions(planner, cache, [n], [[c[0]] for c in cuts], lambda ctx, spans: part.forward(rows_of([x], spans), ctx, 0))
    for i in range(n):
        count = min(window, i + 1)
        first = i - count + 1
        want_one = 0.5 * count / (count + 3.0)
        want_pos = 0.5 * sum(range(first, i + 1)) / (count + 3.0)
        assert abs(float(got[i, 0]) - want_one) < 1e-5 and abs(float(got[i, 1]) - want_pos) < 1e-3 * max(1.0, want_pos), \
            f"position {i}: saw {float(got[i, 0]):.6f}, {float(got[i, 1]):.4f}; {count} keys from {first} give {want_one:.6f}, {want_pos:.4f}"


# --------------------------------------------------------------------------- attention over cached latents
def latent_part(dtype, heads, dim, rot_dim, vdim, rank, r, own=True, scale=0.25, seed=0, max_seq_len=256):
    from logssms_b200.config.specs import LatentAttentionSpec
    from logssms_b200.parts import LatentAttention
    spec = LatentAttentionSpec(WIDTH, heads, dim, rot_dim, vdim, rank, scale, None, rope_spec(rot_dim, r), EPS, pairing="neighbours",
                               sink=True, head_gate=True, own_latents=own)
    part = LatentAttention(spec, perturb_init=True)
    stored = give_weights(part, dtype, seed=seed)
    part.setup(runtime(dtype, max_seq_len=max_seq_len))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": r}
    return part, stored, m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, rot_dim, vdim, rank, r, reader", [
    (3, 24, 16, 8, 32, rot(16, 10000.0, (4.0, 64, 8.0, 1.0)), (2, 8, 24)), (4, 16, 16, 16, 64, rot(16, 30000.0, (2.0, 16, 4.0, 0.5)), (4, 16, 16)),
    (1, 1, 2, 1, 3, rot(2, 50.0), (1, 2, 1)), (3, 5, 6, 7, 11, rot(6, 3000.0, (8.0, 20, 4.0, 1.0)), (5, 3, 9)),
    (16, 8, 16, 8, 32, rot(8, 100.0), (2, 8, 8)), (5, 8, 32, 24, 64, rot(32, 40000.0, (4.0, 1024, 16.0, 2.0)), (7, 4, 4))])
def test_latent_attention_and_a_reader_of_its_cache(dtype, heads, dim, rot_dim, vdim, rank, r, reader):
    if vdim == 1 and dtype == torch.bfloat16:
        pytest.skip("sizes of 1 are covered in float32")
    part, stored, m = latent_part(dtype, heads, dim, rot_dim, vdim, rank, r, seed=heads + rank)
    rh, rdim, rv = reader
    part2, stored2, m2 = latent_part(dtype, rh, rdim, rot_dim, rv, rank, r, own=False, seed=rank)
    assert "dkv" not in stored2 and part2.cache_needs() == part.cache_needs()
    sharp = 4.0 if dtype == torch.float32 else 1.5
    stored["q"], stored2["q"] = stored["q"] * sharp, stored2["q"] * sharp
    rebind(part, stored, dtype)
    rebind(part2, stored2, dtype)
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3)
    xs = inputs(LENGTHS, WIDTH, dtype, seed=2)
    ys = inputs(LENGTHS, WIDTH, dtype, seed=3)        # the reader sees other inputs (another layer's stream) and the same cache

    def run(ctx, spans):
        a = part.forward(rows_of(xs, spans), ctx, 0)
        b = part2.forward(rows_of(ys, spans), ctx, 0, writes_cache=False)
        return torch.cat([a, b], 1)
    for _ in range(2):
        got = step_in_portions(planner, cache, LENGTHS, CUTS, run)
        for x, y, g in zip(xs, ys, got):
            c, kr = P.latent_kv(x.double(), f64(stored), m, EPS)
            close(g[:, :WIDTH], P.latent_attention(x.double(), f64(stored), m, EPS, c, kr), dtype)
            close(g[:, WIDTH:], P.latent_attention(y.double(), f64(stored2), m2, EPS, c, kr), dtype)


def test_a_reader_refuses_to_write():
    part, _, _ = latent_part(torch.float32, 2, 8, 8, 8, 16, rot(8, 100.0), own=False)
    cache, planner = cache_for([part.cache_needs()], torch.float32, max_requests=2)
    with pytest.raises(ValueError, match="reads another layer's cache"):
        step_in_portions(planner, cache, [4], [[4]], lambda ctx, spans: part.forward(torch.zeros(4, WIDTH, device="cuda"), ctx, 0))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_among_hundreds(dtype):
    """600 tokens over pages of 16 whose last 40 inputs are nearly token 5's (scaled up): what the softmax does with a key
    hundreds of positions and dozens of pages back, in a long prompt portion, a shorter one and decoded tokens, is the
    plain model's."""
    n = 600
    part, stored, m = latent_part(dtype, 2, 16, 16, 8, 32, None, seed=9, max_seq_len=640)
    rebind(part, stored, dtype)
    x = inputs([n], WIDTH, dtype, seed=4)[0]
    x[5] = x[5] * 3
    x[-40:] = x[5] + 0.05 * x[-40:]
    cache, planner = cache_for([part.cache_needs()], dtype, num_pages=48, max_requests=2, max_seq_len=640)
    cuts = [[400], [150], [10]] + [[1]] * 40
    (got,) = step_in_portions(planner, cache, [n], cuts, lambda ctx, spans: part.forward(rows_of([x], spans), ctx, 0))
    c, kr = P.latent_kv(x.double(), f64(stored), m, EPS)
    close(got, P.latent_attention(x.double(), f64(stored), m, EPS, c, kr), dtype)


# --------------------------------------------------------------------------- gated delta rule, one decay per head
def delta_part(dtype, heads, kv_heads, dim, vdim, conv, seed=0):
    from logssms_b200.config.specs import GatedDeltaSpec
    from logssms_b200.parts import GatedDelta
    part = GatedDelta(GatedDeltaSpec(WIDTH, heads, kv_heads, dim, vdim, conv, EPS), perturb_init=True)
    stored = give_weights(part, dtype, seed=seed)
    return part, stored, {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, conv", [
    (4, 2, 16, 24, 3), (2, 2, 32, 16, 4), (3, 3, 8, 136, 1), (6, 1, 24, 8, 2), (1, 1, 2, 1, 2), (2, 1, 40, 72, 4),
    (3, 1, 12, 5, 5), (2, 2, 72, 12, 8), (2, 1, 64, 32, 3), (2, 1, 136, 40, 3), (1, 1, 272, 8, 2)])
def test_gated_delta_in_portions(dtype, heads, kv_heads, dim, vdim, conv):
    if vdim == 1 and dtype == torch.bfloat16:
        pytest.skip("a norm over one channel is a sign")
    part, stored, m = delta_part(dtype, heads, kv_heads, dim, vdim, conv, seed=heads + dim)
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3)
    xs = inputs(LENGTHS, WIDTH, dtype, seed=1)
    for _ in range(2):
        got = step_in_portions(planner, cache, LENGTHS, CUTS, lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, P.delta_rule(x.double(), f64(stored), m, EPS), dtype)


def test_gated_delta_keeps_what_it_wrote_long_ago():
    """Decays of nearly one (A_log very negative): what token 0 wrote is still read 500 tokens later, through a prompt in two
    long portions and decoded tokens."""
    dtype = torch.float32
    part, stored, m = delta_part(dtype, 2, 1, 16, 8, 2, seed=5)
    stored["A_log"] = torch.full_like(stored["A_log"], -9.0)
    stored["b"] = stored["b"] * 0.0
    stored["b"][:, 0] = 8.0                                   # the write gate follows input column 0
    rebind(part, stored, dtype)
    n = 520
    x = inputs([n], WIDTH, dtype, seed=6)[0]
    x[:, 0] = -3.0
    x[0, 0] = 3.0                                             # only token 0 writes much
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=2, max_seq_len=640)
    cuts = [[300], [200]] + [[1]] * 20
    (got,) = step_in_portions(planner, cache, [n], cuts, lambda ctx, spans: part.forward(rows_of([x], spans), ctx, 0))
    want = P.delta_rule(x.double(), f64(stored), m, EPS)
    close(got, want, dtype)
    silent = x.clone()
    silent[0, 0] = -3.0
    other = P.delta_rule(silent.double(), f64(stored), m, EPS)
    assert float((other[-1] - want[-1]).abs().max()) > 0.05 * float(want[-1].abs().max())   # the first token's write still matters at the end


# --------------------------------------------------------------------------- the block and its small kernels
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ff", [40, None])
def test_block_norms_its_sublayers_outputs(dtype, ff):
    from logssms_b200.config.specs import GatedDeltaSpec, GLUSpec, MixerSlot, NormSpec, OutNormBlockSpec
    from logssms_b200.ops import kernels as K
    from logssms_b200.parts import OutNormStreamBlock
    norm = NormSpec(WIDTH, EPS, param_name="")
    spec = OutNormBlockSpec("", MixerSlot(GatedDeltaSpec(WIDTH, 2, 1, 8, 16, 3, EPS), "mix."), norm, "norm1",
                            None if ff is None else GLUSpec(WIDTH, ff, "silu"), "mlp.", None if ff is None else norm, "norm2")
    block = OutNormStreamBlock(spec, perturb_init=True)
    stored = give_weights(block, dtype, seed=7)
    cache, planner = cache_for([block.cache_needs()], dtype, max_requests=3)
    xs = inputs(LENGTHS, WIDTH, dtype, seed=8)

    def run(ctx, spans):
        rows = rows_of(xs, spans)
        out, rest = block.forward(K.StreamRows(rows.float().contiguous(), rows), None, ctx, 0)
        assert rest is None and out.f32.dtype == torch.float32 and out.act.dtype == dtype
        assert torch.equal(out.act.float(), out.f32.to(dtype).float())             # the rounded copy is the stream, rounded
        return out.f32
    got = step_in_portions(planner, cache, LENGTHS, CUTS, run)
    w = f64(stored)
    for x, y in zip(xs, got):
        h = x.double()
        mix = {k[4:]: v for k, v in w.items() if k.startswith("mix.")}
        h = h + P.rms_norm(P.delta_rule(h, mix, {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 16}, EPS), w["norm1"], EPS)
        if ff is not None:
            h = h + P.rms_norm(P.dense_ff(h, {k[4:]: v for k, v in w.items() if k.startswith("mlp.")}), w["norm2"], EPS)
        close(y, h, dtype)


@pytest.mark.parametrize("width", [12, 16, 1, 64])                 # multiples of 8 take the form of 16-byte words in bfloat16
@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gate_kernel(dtype, width):
    from logssms_b200.ops import kernels as K
    g = torch.Generator().manual_seed(0)
    o = torch.randn(37, 5 * width, generator=g).to(dtype).cuda()
    wide = torch.randn(37, 9, generator=g).cuda()
    for gate in (wide[:, 2:7], wide.to(dtype)[:, 2:7]):                        # float32 and activation-dtype logits, column views
        want = (o.double().view(37, 5, width) * torch.sigmoid(gate.double())[:, :, None]).view(37, 5 * width)
        close(K.head_gate(o.clone(), gate, 5), want, dtype)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("dtype", DTYPES)
def test_convolution_without_activation(dtype, taps):
    """The short convolution followed by nothing (the attention's), with one tap too, in portions through state slots."""
    from logssms_b200.cache import CacheNeeds, StateNeed
    from logssms_b200.ops import kernels as K
    C = 24
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    xs = inputs(LENGTHS, C, dtype, seed=2)
    needs = CacheNeeds(states=(StateNeed("conv", (C, taps - 1), None),) if taps > 1 else ())
    cache, planner = cache_for([needs], dtype, max_requests=3)

    def run(ctx, spans):
        state = ctx.cache.states[0]["conv"] if taps > 1 else None
        return K.causal_conv1d(rows_of(xs, spans), w.cuda(), None, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests,
                               ctx.max_len, (C, C), (1.0, 1.0, 1.0), activation="none")
    got = step_in_portions(planner, cache, LENGTHS, CUTS, run)
    for x, y in zip(xs, got):
        close(y, P.short_conv(x.double(), w.double()), dtype, tol=1e-5 if dtype == torch.float32 else 1e-2)
