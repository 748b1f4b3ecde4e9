"""Satavik on the GPU against the plain implementation (tests/plain_satavik.py): every mechanism alone through its
part or kernel, then whole models through the engine's step function, decode graph and generation loop, cut and
batched in every way a server would."""
import math

import numpy as np
import pytest
import torch

import plain_satavik as P
import satavik_cases as C
from helpers import TOL, host, rel_error

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [("float32", torch.float32), ("bfloat16", torch.bfloat16)]
PART_TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
SHARP_TOL = {torch.float32: 2e-5, torch.bfloat16: 5e-2}
"""For the tests whose weights make one score stand out: such sharp maps amplify the rounding of bfloat16 keys, and what
the tests decide (a key seen or not) moves the output by more than 0.2."""


def _runtime(dtype, max_length=1024):
    from etalii.dllm_b200.engine.runtime import Runtime

    return Runtime(DEV, dtype, max_length)


def _f64(weights):
    return {k: v.to(P.F64) for k, v in weights.items()}


def _bf16(generator, rows, cols, gain=1.0):
    return (torch.randn(rows, cols, generator=generator) * gain / math.sqrt(cols)).to(torch.bfloat16)


# ---- the small kernels ------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("width", [72, 1000, 4100])
def test_output_norm_adds_the_normed_rows(width):
    from etalii.dllm_b200.kernels import ops

    g = torch.Generator().manual_seed(width)
    x, y = torch.randn(7, width, generator=g), 3.0 * torch.randn(7, width, generator=g) + 0.5
    w = 1 + 0.1 * torch.randn(width, generator=g)
    residual = x.to(DEV)
    ops.norm_add_residual(residual, y.to(DEV), w.to(DEV), 3e-4)
    want = x.to(P.F64) + P.rms(y.to(P.F64), 3e-4) * w.to(P.F64)
    assert rel_error(host(residual), want.numpy()) <= 2e-6


@pytest.mark.parametrize("count", [1, 7, 4096, 100001])
def test_the_stream_rounded_to_the_activation_type(count):
    from etalii.dllm_b200.kernels import ops

    x = torch.randn(count, device=DEV)
    out = torch.empty(count, dtype=torch.bfloat16, device=DEV)
    ops.cast_rows(out, x)
    assert torch.equal(out, x.to(torch.bfloat16))


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("experts,top,width", [(5, 3, 96), (2, 2, 64), (40, 1, 200), (256, 16, 72)])
def test_router_choices_and_weights(name, dtype, experts, top, width):
    from etalii.dllm_b200.kernels import ops

    g = torch.Generator().manual_seed(experts)
    router = _bf16(g, experts, width, 4.0).float()
    bias = torch.randn(experts, generator=g).to(torch.bfloat16).float()
    x = torch.randn(37, width, generator=g).to(dtype)
    chosen = torch.empty(37, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(37, top, device=DEV)
    ops.moe_route(chosen, weights, x.to(DEV), router.to(DEV), bias.to(DEV), top)
    want_chosen, want_weights = P.route({"router": router.to(P.F64), "router.b": bias.to(P.F64)}, x.to(P.F64), top)
    assert chosen.cpu().tolist() == want_chosen.tolist()
    assert rel_error(host(weights), want_weights.numpy()) <= 1e-5


def test_router_ties_go_to_the_lower_expert_and_the_bias_decides():
    from etalii.dllm_b200.kernels import ops

    router = torch.zeros(6, 8)
    router[:, 0] = 1.0  # every expert gets the same logit from x ...
    bias = torch.tensor([0.0, 0.5, 0.0, 0.5, 0.0, 0.0])  # ... and the bias lifts experts 1 and 3
    x = torch.ones(3, 8)
    chosen = torch.empty(3, 3, dtype=torch.int32, device=DEV)
    weights = torch.empty(3, 3, device=DEV)
    ops.moe_route(chosen, weights, x.to(DEV), router.to(DEV), bias.to(DEV), 3)
    assert chosen.cpu().tolist() == [[1, 3, 0]] * 3
    e = math.exp(-0.5)
    assert np.allclose(host(weights), [[1 / (2 + e), 1 / (2 + e), e / (2 + e)]] * 3, atol=1e-6)


# ---- the parts --------------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5, 70, 333])
@pytest.mark.parametrize("experts,top,ff,shared", [(5, 3, 24, 40), (3, 1, 20, 0), (2, 2, 8, 8), (40, 2, 136, 0)])
def test_mixture_part(name, dtype, rows, experts, top, ff, shared):
    from etalii.dllm_b200.kernels import ops
    from etalii.dllm_b200.parts import PartSpec, build_part
    from etalii.dllm_b200.parts.norm import StreamOperand

    rt = _runtime(dtype)
    width = 72
    shared_spec = PartSpec("clamped_glu", {"hidden_size": width, "intermediate_size": shared, "limit": 0.6}) \
        if shared else None
    part = build_part("feed_forward", PartSpec("clamped_glu_experts", {
        "hidden_size": width, "intermediate_size": ff, "experts": experts, "top": top, "limit": 0.9,
        "shared": shared_spec}))
    g = torch.Generator().manual_seed(rows + experts)
    weights = {"router": _bf16(g, experts, width, 4.0), "router_bias": torch.randn(experts, generator=g).to(torch.bfloat16)}
    for e in range(experts):
        weights.update({f"e{e}.gate": _bf16(g, ff, width, 1.5), f"e{e}.up": _bf16(g, ff, width, 1.5),
                        f"e{e}.down": _bf16(g, width, ff)})
    if shared:
        weights.update({"shared.gate": _bf16(g, shared, width, 1.5), "shared.up": _bf16(g, shared, width, 1.5),
                        "shared.down": _bf16(g, width, shared)})
    part.bind(weights, rt)
    x = torch.randn(rows, width, generator=g).to(dtype).float()  # (the stream holds values of the activation type)
    plain_w = _f64({k.replace("router_bias", "router.b"): v for k, v in weights.items()})
    mlp = {"expert": {"limit": 0.9}, "router": {"top": top}, "shared": {"limit": 0.6} if shared else None}
    want = P.mixture(plain_w, mlp, x.to(P.F64)).numpy()
    stored = torch.full((rows, width), 7.0, device=DEV)
    part.forward(StreamOperand(x.to(DEV), rt), stored, None, rt, epilogue=ops.EPI_STORE_F32)
    assert rel_error(host(stored), want) <= PART_TOL[dtype]
    added = torch.ones(rows, width, device=DEV)
    part.forward(x.to(dtype).to(DEV), added, None, rt)  # the rounded activations, added into a stream
    assert rel_error(host(added), 1 + want) <= PART_TOL[dtype]


class MixerHarness:
    """A differential-attention part with a cache of its own and sequences that are fed in pieces."""

    def __init__(self, part, dtype, sequences, pages=48):
        from etalii.dllm_b200.cache.paged import PagedCache
        from etalii.dllm_b200.engine.batch import BatchBuffers

        self.cache = PagedCache([part.cache_need()], 64 * pages, 1024, dtype=dtype, device=DEV)
        self.view = self.cache.kv_view(0)
        self.part, self.buffers = part, BatchBuffers(DEV)
        self.slots = self.cache.acquire(sequences)

    def step(self, rt, which, pieces, width):
        from etalii.dllm_b200.kernels import ops

        slots = [self.slots[i] for i in which]
        starts = []
        for slot, piece in zip(slots, pieces):
            self.cache.reserve(slot, piece.shape[0])
            starts.append(self.cache.length(slot))
        self.cache.sync_tables()
        batch = self.buffers.fill(slots, [[0] * p.shape[0] for p in pieces], starts, [[] for _ in pieces])
        h = torch.cat(pieces).to(rt.dtype).to(DEV).contiguous()
        out = torch.zeros(h.shape[0], width, device=DEV)
        self.part.forward(h, out, batch, self.view, rt, epilogue=ops.EPI_STORE_F32)
        for slot, piece in zip(slots, pieces):
            self.cache.advance(slot, piece.shape[0])
        rows, at = [], 0
        for piece in pieces:
            rows.append(host(out[at:at + piece.shape[0]]))
            at += piece.shape[0]
        return rows


def _feed(harness, rt, sequences, schedule, width):
    at = [0] * len(sequences)
    got = [[] for _ in sequences]
    for step in schedule:
        which = [i for i, _ in step]
        pieces = [sequences[i][at[i]:at[i] + n] for i, n in step]
        for (i, n), rows in zip(step, harness.step(rt, which, pieces, width)):
            got[i].append(rows)
            at[i] += n
    assert all(a == s.shape[0] for a, s in zip(at, sequences))
    return [np.concatenate(g) for g in got]


def _mixer(width, p, eps=1e-5):
    from etalii.dllm_b200.parts import PartSpec, build_part

    position = PartSpec("rotary", {"head_dim": p["dim"], "theta": p["rot"]["base"], "rotary_dim": p["rot"]["dims"],
                                   "pairing": "halves"}) if p["rot"]["dims"] else None
    return build_part("mixer", PartSpec("differential_attention", {
        "hidden_size": width, "num_heads": p["heads"], "num_kv_heads": p["kv_heads"], "dim": p["dim"],
        "vdim": p["vdim"], "scale": p["scale"], "diff": p["diff"], "eps": eps, "softcap": p["softcap"],
        "chunk": p["mask"]["size"], "position": position}))


def _mixer_weights(g, width, p):
    w = {"q": _bf16(g, p["heads"] * 2 * p["dim"], width, 1.5), "k": _bf16(g, p["kv_heads"] * 2 * p["dim"], width, 1.5),
         "v": _bf16(g, p["kv_heads"] * p["vdim"], width, 1.5), "g": _bf16(g, p["heads"], width, 2.0),
         "o": _bf16(g, width, p["heads"] * p["vdim"]),
         "q_norm": (1.5 + 0.4 * torch.randn(p["dim"], generator=g)).to(torch.bfloat16),
         "k_norm": (1.5 + 0.4 * torch.randn(p["dim"], generator=g)).to(torch.bfloat16)}
    for name in ("lq1", "lk1", "lq2", "lk2"):
        w[name] = (0.4 * torch.randn(p["dim"], generator=g)).to(torch.bfloat16)
    return w


def _plain_names(w):
    return _f64({k.replace("q_norm", "q.norm").replace("k_norm", "k.norm"): v for k, v in w.items()})


def _plain_mixer(w, p, h, eps=1e-5):
    cache = {}
    P.project_keys(_plain_names(w), p, h.to(P.F64), 0, eps, cache)
    return P.differential_attention(_plain_names(w), p, h.to(P.F64), 0, eps, cache).numpy()


SCHEDULE = [[(0, 70), (1, 2), (2, 17)], [(0, 1), (1, 1), (2, 1)], [(0, 1), (1, 1), (2, 1)], [(0, 2), (2, 65)],
            [(0, 1), (2, 1)], [(2, 1)]]
LENGTHS = [75, 4, 86]
SHAPES = {
    "wide_values": dict(heads=6, kv_heads=2, dim=16, vdim=40, rot=dict(base=1e4, dims=8), scale=0.3, softcap=20.0,
                        diff=0.25, mask=dict(size=48)),
    "no_pieces": dict(heads=2, kv_heads=1, dim=20, vdim=12, rot=dict(base=50.0, dims=0), scale=0.5, softcap=4.0,
                      diff=0.6, mask=dict(size=5)),
    "one_chunk": dict(heads=4, kv_heads=4, dim=64, vdim=128, rot=dict(base=1e6, dims=64), scale=0.125, softcap=50.0,
                      diff=0.1, mask=dict(size=4096)),
}


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_differential_attention_part_in_pieces(name, dtype, shape):
    """Three sequences fed as a server would: a prompt portion that crosses a page border, portions of two tokens,
    single tokens beside neighbours, a sequence that ends early; against the plain mixer on each whole sequence."""
    rt = _runtime(dtype)
    p, width = SHAPES[shape], 72
    part = _mixer(width, p)
    g = torch.Generator().manual_seed(len(shape))
    weights = _mixer_weights(g, width, p)
    part.bind(weights, rt)
    sequences = [torch.randn(n, width, generator=g).to(dtype).float() for n in LENGTHS]
    got = _feed(MixerHarness(part, dtype, 3), rt, sequences, SCHEDULE, width)
    for rows, h in zip(got, sequences):
        assert rel_error(rows, _plain_mixer(weights, p, h)) <= PART_TOL[dtype]
    assert abs(part.weight - P.difference_weight(_plain_names(weights), p["diff"])) <= 1e-6


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("chunk", [100, 64, 37])
@pytest.mark.parametrize("back", [0, 1, 2])
def test_a_key_at_the_edge_of_a_chunk_counts_only_from_inside(name, dtype, chunk, back):
    """One key is made to take all the weight of whoever sees it (its key and the later queries are one strong
    direction). It stands at the first place of a chunk, or one or two places before: the tokens of the chunk must
    see it in the first case and must not in the others; the same for a token decoded alone after the prompt. The
    outputs with and without that key differ by far more than the tolerance."""
    rt = _runtime(dtype)
    width = 48
    p = dict(heads=2, kv_heads=1, dim=32, vdim=24, rot=dict(base=1e4, dims=0), scale=1.0, softcap=30.0, diff=0.3,
             mask=dict(size=chunk))
    part = _mixer(width, p)
    g = torch.Generator().manual_seed(chunk + back)
    weights = _mixer_weights(g, width, p)
    # Map 1's queries read the first half of h and its keys the second half through the same matrix: a token whose
    # second half is u is the one key that the queries of tokens whose first half is u point at (vectors are normed,
    # so only directions count); values read all of h, so that key's value is like no other.
    half = width // 2
    reads = _bf16(g, 32, half, 6.0)
    nothing = torch.zeros(32, half, dtype=torch.bfloat16)
    weights["k"] = torch.cat([torch.cat([nothing, reads], dim=1), _bf16(g, 32, width, 1.5)])
    weights["q"] = torch.cat([torch.cat([reads, nothing], dim=1), _bf16(g, 32, width, 1.5)] * 2)
    part.bind(weights, rt)
    start = 2 * chunk  # the third chunk's first position
    n = start + 9
    h = torch.randn(n + 1, width, generator=g)
    special = start - back
    u = torch.randn(half, generator=g)
    h[special, half:] = u
    for row in range(start + 1, n + 1):
        h[row, :half] = u + 0.05 * torch.randn(half, generator=g)
    h = h.to(dtype).float()
    got = _feed(MixerHarness(part, dtype, 1), rt, [h], [[(0, n)], [(0, 1)]], width)[0]
    want = _plain_mixer(weights, p, h)
    without = h.clone()
    without[special] = 0.0
    other = _plain_mixer(weights, p, without)
    for row in (start + 1, n - 1, n):  # in the prompt, and the token decoded alone
        sees = back == 0
        assert (rel_error(want[row], other[row]) > 0.2) == sees  # the test's premise
        assert rel_error(got[row], want[row]) <= SHARP_TOL[dtype]


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 63, 64, 65, 127, 128, 300])
def test_a_far_key_among_hundreds(name, dtype, far):
    """One key far back, at and around page borders, takes the weight of the last tokens of a chunk of 1000 positions,
    in the prompt and in a token decoded alone."""
    rt = _runtime(dtype)
    width = 48
    p = dict(heads=3, kv_heads=3, dim=16, vdim=16, rot=dict(base=1e6, dims=4), scale=1.0, softcap=40.0, diff=0.2,
             mask=dict(size=1000))
    part = _mixer(width, p)
    g = torch.Generator().manual_seed(20 + far)
    weights = _mixer_weights(g, width, p)
    # (as above: queries read the first half of h, keys the second half, through the same matrix)
    half = width // 2
    reads = _bf16(g, 3 * 2 * 16, half, 6.0).float().view(6, 16, half)
    reads[:, :4] *= 0.2  # (the rotated places weigh little here, so no angle can turn the far score round)
    reads = reads.reshape(96, half).to(torch.bfloat16)
    nothing = torch.zeros(96, half, dtype=torch.bfloat16)
    weights["q"], weights["k"] = torch.cat([reads, nothing], dim=1), torch.cat([nothing, reads], dim=1)
    part.bind(weights, rt)
    n = 420
    h = torch.randn(n + 1, width, generator=g)
    u = torch.randn(half, generator=g)
    h[far, half:] = u
    h[n - 1, :half] = h[n, :half] = u
    h = h.to(dtype).float()
    got = _feed(MixerHarness(part, dtype, 1), rt, [h], [[(0, n)], [(0, 1)]], width)[0]
    want = _plain_mixer(weights, p, h)
    without = h.clone()
    without[far] = 0.0
    other = _plain_mixer(weights, p, without)
    for row in (n - 1, n):
        assert rel_error(want[row], other[row]) > 0.2  # the test's premise: that key matters
        assert rel_error(got[row], want[row]) <= SHARP_TOL[dtype]


@pytest.mark.parametrize("name,dtype", DTYPES)
def test_many_sequences_decode_side_by_side(name, dtype):
    """Forty sequences of unequal lengths, then three steps of one token each (the warp-per-pair launch shape)."""
    rt = _runtime(dtype)
    p, width = SHAPES["wide_values"], 72
    part = _mixer(width, p)
    g = torch.Generator().manual_seed(77)
    weights = _mixer_weights(g, width, p)
    part.bind(weights, rt)
    lengths = [4 + (7 * i) % 60 for i in range(40)]
    sequences = [torch.randn(n, width, generator=g).to(dtype).float() for n in lengths]
    schedule = [[(i, n - 3) for i, n in enumerate(lengths)]] + [[(i, 1) for i in range(40)]] * 3
    got = _feed(MixerHarness(part, dtype, 40, pages=96), rt, sequences, schedule, width)
    for rows, h in zip(got, sequences):
        assert rel_error(rows, _plain_mixer(weights, p, h)) <= PART_TOL[dtype]


# ---- whole models through the engine ------------------------------------------------------------------------------------


class Case:
    def __init__(self, case, seed=1):
        self.config = C.CASES[case]()
        self.tensors = C.random_weights(self.config, seed)
        self._memo = {}

    def logits(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = P.forward(self.config, self.tensors, list(tokens)).numpy()
        return self._memo[key]


_CASES = {}


def _case(name) -> Case:
    if name not in _CASES:
        _CASES[name] = Case(name)
    return _CASES[name]


def _run(engine, prompts, schedule):
    """Feeds `prompts` by `schedule` (steps of (prompt, count)); a prompt's slot is given back with its last token.
    Returns every position's logits per prompt."""
    at = [0] * len(prompts)
    slots = {}
    rows = [[] for _ in prompts]
    for step in schedule:
        for i, _ in step:
            if i not in slots:
                slots[i] = engine.open(1)[0]
        pieces = [prompts[i][at[i]:at[i] + n] for i, n in step]
        out = host(engine.step([slots[i] for i, _ in step], pieces, [list(range(len(p))) for p in pieces]))
        engine.check()
        offset = 0
        for (i, n) in step:
            rows[i].append(out[offset:offset + n])
            offset += n
            at[i] += n
            if at[i] == len(prompts[i]):
                engine.close([slots.pop(i)])
    assert not slots
    return [np.concatenate(r) for r in rows]


def _compare(case, got, prompts, dtype_name):
    """float32: every logit of every position within the tolerance. bfloat16: rounding upstream can move a router logit
    past its neighbour, and the token then runs another expert than the plain model's; so there 9 of 10 positions
    must be within the tolerance and the median position within a third of it. (What a lost key, a wrong chunk or a
    stale page does is decided in float32, where the same schedules run through the same cache and step function.)"""
    errors = []
    for rows, tokens in zip(got, prompts):
        want = case.logits(tokens)
        assert rows.shape == want.shape
        errors += list(np.abs(rows - want).max(axis=1) / np.abs(want).max())
    errors = np.sort(np.asarray(errors))
    if dtype_name == "float32":
        assert errors[-1] <= TOL[dtype_name]
    else:
        assert errors[int(0.9 * (len(errors) - 1))] <= TOL[dtype_name] and np.median(errors) <= TOL[dtype_name] / 3


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_whole_prompts_alone_and_as_one_batch(name, dtype_name):
    case = _case(name)
    engine = C.make_engine(case.config, case.tensors, dtype_name)
    prompts = C.tokens_for(case.config, [1, 2, 70, 131, 5])
    alone = _run(engine, prompts, [[(i, len(p))] for i, p in enumerate(prompts)])
    _compare(case, alone, prompts, dtype_name)
    together = _run(engine, prompts, [[(i, len(p)) for i, p in enumerate(prompts)]])
    _compare(case, together, prompts, dtype_name)
    if dtype_name == "float32":  # batch mates change nothing beyond rounding; in float32 that is very little
        assert all(rel_error(a, b) <= 1e-5 for a, b in zip(alone, together))
    engine.cache.check()


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_portions_and_single_tokens(name, dtype_name):
    """One prompt cut into portions of 64, 2, 65, 3 and 1, 1, ...: the pieces cross page and chunk borders and end in
    token-by-token decoding; then the first tokens one by one from an empty cache."""
    case = _case(name)
    engine = C.make_engine(case.config, case.tensors, dtype_name)
    prompt = C.tokens_for(case.config, [150], seed=6)[0]
    schedule = [[(0, 64)], [(0, 2)], [(0, 65)], [(0, 3)]] + [[(0, 1)]] * 16
    _compare(case, _run(engine, [prompt], schedule), [prompt], dtype_name)
    schedule = [[(0, 1)]] * 5 + [[(0, 145)]]
    _compare(case, _run(engine, [prompt], schedule), [prompt], dtype_name)
    engine.cache.check()
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_unequal_batches_early_finishers_and_slots_used_again(name, dtype_name):
    """Requests of unequal length start together and decode together; the shorter ones end earlier and give their
    slots and pages back; later requests take those slots and pages (which still hold the old keys) and run beside
    the survivors."""
    case = _case(name)
    engine = C.make_engine(case.config, case.tensors, dtype_name, max_tokens=64 * 8, max_slots=4)
    prompts = C.tokens_for(case.config, [40, 9, 75, 30, 12], seed=8)
    schedule = [[(0, 30), (1, 6), (2, 66)]]
    schedule += [[(0, 1), (1, 1), (2, 1)]] * 3          # request 1 ends here
    schedule += [[(0, 1), (2, 1)]] * 6                  # request 2 ends here
    schedule += [[(3, 25), (4, 10)]]                    # two new requests take the freed slots
    schedule += [[(0, 1), (3, 1), (4, 1)]]              # ... and decode beside the survivor
    schedule += [[(3, 1), (4, 1)], [(3, 3)]]
    got = _run(engine, prompts, schedule)
    _compare(case, got, prompts, dtype_name)
    engine.cache.check()
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_pages_behind_a_chunk_stay_while_a_borrowing_layer_still_reads_them(dtype_name):
    """A layer with chunks of 70 positions lends its keys to a layer with chunks of 1000. A request passes position
    140; what the lender no longer needs, the borrower still reads, so those pages must not go to the second request,
    which starts right then and takes whatever pages are free (the most recently freed first). The first layer's
    entry (chunks of 48 and 33) does give pages back, and they are used again."""
    case = _case("borrowed")
    engine = C.make_engine(case.config, case.tensors, dtype_name, max_tokens=64 * 10, max_slots=2)
    prompts = C.tokens_for(case.config, [150, 60], seed=14)
    schedule = [[(0, 145)], [(1, 60)]] + [[(0, 1)]] * 5
    _compare(case, _run(engine, prompts, schedule), prompts, dtype_name)
    engine.cache.check()
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_long_decoding_through_the_decode_graph(dtype_name):
    """A hundred and fifty single-token steps of three sequences as the generation loop runs them (one captured graph
    replayed): they pass several chunk borders, and pages of finished chunks go back to the pool on the way. Then
    the last step's logits against the plain implementation on the whole history."""
    case = _case("borrowed")
    engine = C.make_engine(case.config, case.tensors, dtype_name, decode_logits=True)
    prompts = C.tokens_for(case.config, [7, 20, 66], seed=9)
    slots = engine.open(3)
    first = host(engine.step(slots, prompts)).argmax(axis=1).tolist()
    chosen = engine.decode(slots, first, 150)
    histories = [p + [f] + [step[i] for step in chosen] for i, (p, f) in enumerate(zip(prompts, first))]
    graph_logits = host(engine.last_decode_graph.logits)  # of the last step: history without its last token
    for i, history in enumerate(histories):
        want = case.logits(history[:-1])[-1]
        assert rel_error(graph_logits[i], want) <= TOL[dtype_name]
        if dtype_name == "float32":
            assert int(np.argmax(want)) == history[-1]
    engine.close(slots)
    engine.cache.check()


def test_greedy_generation_through_the_generation_loop():
    """`Engine.generate` (batches planned by the scheduler, prompt step, decode graphs, early finishers) gives the
    tokens the plain implementation chooses greedily, in float32."""
    from etalii.dllm_b200 import SamplingOptions

    case = _case("narrow")
    engine = C.make_engine(case.config, case.tensors, "float32")
    prompts = C.tokens_for(case.config, [3, 18, 70], seed=10)
    results = engine.generate(prompts, 12, SamplingOptions(), ignore_eos=True)
    for prompt, result in zip(prompts, results):
        history = list(prompt)
        for _ in range(12):
            history.append(int(np.argmax(case.logits(history)[-1])))
        assert list(result.tokens) == history[len(prompt):]
    again = engine.generate(prompts[:2], 5, SamplingOptions(), ignore_eos=True)  # the slots are used again
    assert [list(r.tokens) for r in again] == [list(r.tokens)[:5] for r in results[:2]]


def test_sampled_generation_runs_in_bfloat16():
    from etalii.dllm_b200 import SamplingOptions

    case = _case("borrowed")
    engine = C.make_engine(case.config, case.tensors, "bfloat16")
    prompts = C.tokens_for(case.config, [5, 33], seed=11)
    a = engine.generate(prompts, 20, SamplingOptions(temperature=0.8, top_k=20, seed=3), ignore_eos=True)
    b = engine.generate(prompts, 20, SamplingOptions(temperature=0.8, top_k=20, seed=3), ignore_eos=True)
    assert [list(r.tokens) for r in a] == [list(r.tokens) for r in b] and all(len(r.tokens) == 20 for r in a)


def test_trace_replay_and_command_line_on_a_satavik_folder(tmp_path):
    """bin/trace_run and `dllm-b200 generate` as subprocesses on a model folder the library wrote."""
    import json
    import os
    import subprocess
    import sys

    from etalii.dllm_b200.weights.random_init import write_model

    case = _case("narrow")
    folder = write_model(str(tmp_path / "model"), case.config, case.tensors)
    tokens = C.tokens_for(case.config, [20], seed=12)[0]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[17:18], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[18:20], "want": [1]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.split("\n") if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = case.logits(tokens)
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    last = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)
    assert not (out / "1.f32").exists()
    assert rel_error(first, want[[0, 16]]) <= TOL["float32"] and rel_error(last, want[[19]]) <= TOL["float32"]

    tool = [sys.executable, os.path.join(root, "bin", "dllm-b200")]
    done = subprocess.run(tool + ["--model", folder, "info"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and json.loads(done.stdout)["architecture"] == "Satavik"
    prompt = tokens[:9]
    done = subprocess.run(tool + ["--model", folder, "--dtype", "float32", "--cache-tokens", "256", "generate",
                                  "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--ignore-eos"],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    history = list(prompt)
    for _ in range(6):
        history.append(int(np.argmax(case.logits(history)[-1])))
    assert [int(t) for t in done.stdout.split()] == history[len(prompt):]
