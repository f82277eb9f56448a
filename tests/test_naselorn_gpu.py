"""The Naselorn design in the engine against the plain float64 model of ``plain_naselorn.py``: whole prompts,
decoding token by token, portions down to two tokens, batches of unequal requests, pages and slots used again,
keys just inside and just outside a chunk with weights that make one key show, a far token through the lightning
state and through the recurrent unit's state, the convolution's carried inputs, the router's choices and bias, and
greedy generation through ``Engine`` and the command line. float32 path to 2e-4 of the logits' spread, bfloat16
path to a few percent."""
from __future__ import annotations

import numpy as np
import pytest

import naselorn_models as nm
import plain_naselorn as plain

pytestmark = pytest.mark.gpu

LIMIT = {"float32": 2e-4, "bfloat16": 1.5e-1}
TYPICAL = {"float32": 1e-4, "bfloat16": 5e-2}


def spread_error(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: rms of the difference (mean taken off) over the rms of the wanted row (mean taken off)."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean(-1))


def check(got, want, dtype, what, routed=False):
    """``routed``: the model chooses experts. In bfloat16 a token whose best choices lie close together may take
    another expert than in the plain model, and its row (and, fading, the rows after it) then differs by more than
    rounding; one row in twelve (rounded up) may, by at most the row's whole spread. float32 is held to the limit everywhere."""
    err = spread_error(np.asarray(got, dtype=np.float64), want)
    worst = int(np.argmax(err))
    if routed and dtype == "bfloat16":
        assert err[worst] <= 1.0, f"{what}: row {worst} differs by {err[worst]:.3e} of the row's spread"
        assert (err > LIMIT[dtype]).sum() <= -(-len(err) // 12), f"{what}: {(err > LIMIT[dtype]).sum()} rows over the limit"
    else:
        assert err[worst] <= LIMIT[dtype], f"{what}: row {worst} differs by {err[worst]:.3e} of the row's spread"
    assert np.median(err) <= TYPICAL[dtype], f"{what}: half of the rows differ by {np.median(err):.3e} and more"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("naselorn")
    out = {}
    for name, (raw, seed) in nm.CONFIGS.items():
        folder = str(base / name)
        raw, tensors = nm.write_model(folder, raw, seed)
        out[name] = (folder, raw, plain.as_float64(tensors))
    return out


def load(folder, dtype, **kw):
    from celeg_b200.engine.loading import load_model
    args = dict(dtype=dtype, max_requests=4, cache_tokens=1024, max_batched_tokens=512, max_context=512)
    args.update(kw)
    return load_model(folder, **args)


def run_steps(loaded, steps):
    """steps: lists of (request, tokens); every place is wanted. Returns {request: [its logits rows in order]}."""
    from celeg_b200.engine.step import StepEntry
    rows = {}
    for step in steps:
        step = [(name, tokens) for name, tokens in step if len(tokens) > 0]
        entries = [StepEntry(name, list(tokens), list(range(len(tokens)))) for name, tokens in step]
        logits = loaded.step.run(entries, auto_begin=True).cpu().numpy()
        loaded.step.raise_on_device_error()
        at = 0
        for name, tokens in step:
            rows.setdefault(name, []).append(logits[at:at + len(tokens)].copy())
            at += len(tokens)
    return {name: np.concatenate(parts) for name, parts in rows.items()}


def cut(tokens, sizes):
    out, at, i = [], 0, 0
    while at < len(tokens):
        n = sizes[i % len(sizes)]
        out.append(tokens[at:at + n])
        at += n
        i += 1
    return out


def tokens_of(vocab, length, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(nm.CONFIGS))
def test_whole_prompt_then_token_by_token(models, name, dtype):
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 90, 1)
    want = plain.logits(raw, tensors, tokens)
    loaded = load(folder, dtype)
    whole = run_steps(loaded, [[("w", tokens)]])["w"]
    check(whole, want, dtype, f"{name} whole", routed=True)
    loaded.step.end("w")
    steps = [[("d", tokens[:37])]] + [[("d", [t])] for t in tokens[37:]]
    decoded = run_steps(loaded, steps)["d"]
    check(decoded, want, dtype, f"{name} prompt of 37 then token by token", routed=True)
    if dtype == "float32":       # how the prompt is cut changes nothing beyond rounding
        assert np.abs(decoded - whole).max() <= 1e-3 * np.abs(whole).max()


@pytest.mark.parametrize("name", list(nm.CONFIGS))
def test_the_stream_after_every_layer(models, name, tmp_path):
    """A model cut after its n-th layer, with an identity for the final norm's scale and unit rows as its head,
    hands out the stream itself (divided by its root mean square): layer by layer against the plain model."""
    import torch
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 40, 21)
    want = plain.streams(raw, tensors, tokens)
    width = raw["width"]
    for depth in range(1, len(raw["layers"]) + 1):
        short = dict(raw, layers=raw["layers"][:depth], vocab=raw["vocab"])
        kept = {key: torch.from_numpy(value).to(torch.bfloat16) for key, value in tensors.items()
                if not key.startswith("l") or int(key[1:key.index(".")]) < depth}
        kept["final.norm"] = torch.zeros(width, dtype=torch.bfloat16)
        head = torch.zeros((raw["vocab"], width), dtype=torch.bfloat16)
        head[:width] = torch.eye(width)[:raw["vocab"]]
        kept["head"] = head
        cut_folder = str(tmp_path / f"{name}{depth}")
        nm.write_model(cut_folder, short, 0, tensors=kept)
        got = run_steps(load(cut_folder, "float32"), [[("a", tokens)]])["a"][:, :min(width, raw["vocab"])].astype(np.float64)
        stream = want[depth - 1]
        normed = plain.rms_scaled(stream, float(raw["norm"]["eps"]))[:, :got.shape[1]]
        assert np.abs(got - normed).max() <= 5e-5 * np.abs(normed).max(), f"{name} after layer {depth - 1}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(nm.CONFIGS))
def test_portions_of_several_sizes_down_to_two_tokens(models, name, dtype):
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 131, 2)
    want = plain.logits(raw, tensors, tokens)
    loaded = load(folder, dtype)
    for tag, sizes in (("a", [2, 3, 17, 2, 33]), ("b", [16, 16, 1, 15, 48]), ("c", [5, 2, 2, 64])):
        got = run_steps(loaded, [[(tag, part)] for part in cut(tokens, sizes)])[tag]
        check(got, want, dtype, f"{name} in portions of {sizes}", routed=True)
        loaded.step.end(tag)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(nm.CONFIGS))
def test_batches_of_unequal_requests_equal_each_alone(models, name, dtype):
    folder, raw, tensors = models[name]
    requests = {"p": tokens_of(raw["vocab"], 70, 3), "q": tokens_of(raw["vocab"], 23, 4),
                "r": tokens_of(raw["vocab"], 120, 5), "s": tokens_of(raw["vocab"], 9, 6)}
    want = {key: plain.logits(raw, tensors, value) for key, value in requests.items()}
    # portions of some beside single tokens of others; q joins late, s is left out of steps and goes on later
    plan = {"p": [40] + [1] * 30, "q": [0, 0, 2, 19, 1, 1], "r": [3, 50, 1, 1, 1, 62, 1, 1], "s": [1, 0, 0, 1, 0, 5, 2]}
    at = {key: 0 for key in requests}
    steps = []
    for n in range(40):
        step = []
        for key in ("s", "p", "q", "r"):
            sizes = plan[key]
            count = sizes[n] if n < len(sizes) else 1
            count = min(count, len(requests[key]) - at[key])
            if count > 0:
                step.append((key, requests[key][at[key]:at[key] + count]))
                at[key] += count
        if step:
            steps.append(step)
    assert all(at[key] == len(requests[key]) for key in requests)
    got = run_steps(load(folder, dtype), steps)
    for key in requests:
        check(got[key], want[key], dtype, f"{name} request {key} in a batch", routed=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_pages_and_slots_are_used_again(models, name, dtype):
    """Two slots and a pool of 160 positions for six requests one after the other, two live at a time: every
    later request sits in a slot and in pages that an earlier one has left full of its own state."""
    folder, raw, tensors = models[name]
    loaded = load(folder, dtype, max_requests=2, cache_tokens=160)
    lengths = [75, 60, 31, 80, 17, 66]
    for turn in range(3):
        pair = {f"x{2 * turn}": tokens_of(raw["vocab"], lengths[2 * turn], 20 + turn),
                f"y{2 * turn}": tokens_of(raw["vocab"], lengths[2 * turn + 1], 30 + turn)}
        (a, ta), (b, tb) = pair.items()
        steps = [[(a, ta[:20]), (b, tb[:3])], [(a, ta[20:21]), (b, tb[3:])], [(a, ta[21:])]]
        got = run_steps(loaded, steps)
        for key, tokens in pair.items():
            check(got[key], plain.logits(raw, tensors, tokens), dtype, f"turn {turn} request {key}", routed=True)
            loaded.step.end(key)
        loaded.manager.check_invariants()
    assert loaded.manager.free_slots == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_portions_beside_short_ones(models, name, dtype):
    """Portions of hundreds of tokens (the recurrences scan them in segments, the experts' pairs are grouped, the
    chunked mask passes many chunks) beside single tokens and short portions of other requests, from states and
    caches that earlier portions left; positions beyond a thousand in the sinusoid."""
    folder, raw, tensors = models[name]
    long_one, short_one, other = tokens_of(raw["vocab"], 1100, 31), tokens_of(raw["vocab"], 140, 32), tokens_of(raw["vocab"], 400, 33)
    want = {"a": plain.logits(raw, tensors, long_one), "b": plain.logits(raw, tensors, short_one), "c": plain.logits(raw, tensors, other)}
    loaded = load(folder, dtype, cache_tokens=2048, max_batched_tokens=1024, max_context=2048)
    steps = [[("b", short_one[:1]), ("a", long_one[:449])], [("b", short_one[1:2]), ("a", long_one[449:450]), ("c", other[:385])],
             [("b", short_one[2:131]), ("a", long_one[450:1027]), ("c", other[385:])], [("b", short_one[131:]), ("a", long_one[1027:])]]
    got = run_steps(loaded, steps)
    for key in want:
        check(got[key], want[key], dtype, f"{name} request {key} in long portions", routed=True)


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_long_decoding_from_the_first_token(models, name):
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 200, 7)
    got = run_steps(load(folder, "float32"), [[("l", [t])] for t in tokens])["l"]
    check(got, plain.logits(raw, tensors, tokens), "float32", "200 tokens one by one")


# ------------------------------------------------------------------------- one mechanism, made to show
def one_layer_model(tmp_path, layer, seed, mlp=None, **weights):
    raw = nm.single_layer(layer, mlp)
    folder = str(tmp_path / "one")
    raw, tensors = nm.write_model(folder, raw, seed, **weights)
    return folder, raw, plain.as_float64(tensors)


def single_out(bf16, token, column, value=4.0):
    """Column ``column`` of the embedding table becomes zero for every token but ``token``. The tests use even
    columns at the end of the row, where the position vector adds sin(p / 10000^(almost 1)), next to nothing: in a
    model of one layer that input dimension then speaks for this token alone."""
    import torch
    table = bf16["embed"].float().numpy().copy()
    table[:, column] = 0.0
    table[token, column] = value
    bf16["embed"] = torch.from_numpy(table).to(torch.bfloat16)


def set_column(bf16, name, rows, column, values):
    import torch
    matrix = bf16[name].float().numpy().copy()
    matrix[rows, column] = values
    bf16[name] = torch.from_numpy(matrix).to(torch.bfloat16)


def louder(bf16, name, factor):
    import torch
    bf16[name] = (bf16[name].float() * factor).to(torch.bfloat16)


def normed_inputs(raw, bf16, tokens):
    """What the first layer's mixer reads for this sequence, [tokens, width]."""
    tensors = plain.as_float64(bf16)
    return plain.offset_norm(plain.embed(raw, tensors, tokens), tensors["l0.norm1"], float(raw["norm"]["eps"]))


def build_chunk_edge(sizes, chunk, probe, far, length):
    """One side-by-side layer whose right half counts for nothing and in whose left half every head's query of ONE
    token (the probe's, through an input dimension that only this token has) points at the key that ONE other token
    makes at place ``far``. Returns (raw, bf16, sequence with that token, sequence with another in its place)."""
    heads, groups, dim, vdim = sizes
    raw = nm.single_layer(nm.parallel(heads, groups, dim, vdim, chunk, 12, 2, 2, scale=0.2, left_scale=1.5, right_scale=0.0))
    bf16 = nm.make_tensors(raw, 40)
    vocab, width = raw["vocab"], raw["width"]
    key_token, probe_token, other_token = vocab - 1, vocab - 2, vocab - 3
    column, key_column = width - 2, width - 4
    single_out(bf16, probe_token, column)
    single_out(bf16, key_token, key_column)
    changed = np.random.default_rng(8).integers(0, vocab - 3, size=length).tolist()
    changed[probe] = probe_token
    without = list(changed)
    changed[far], without[far] = key_token, other_token
    h = normed_inputs(raw, bf16, changed)
    # (the key token's keys are longer than every other token's, so that no other key lies further along them)
    set_column(bf16, "l0.mix.left.k", slice(0, groups * dim), key_column,
               1.5 * np.random.default_rng(9).normal(size=groups * dim) / h[far][key_column])
    tensors = plain.as_float64(bf16)
    keys = tensors["l0.mix.left.k"] @ h[far] + tensors["l0.mix.left.k.b"]
    for head in range(heads):
        group = head // (heads // groups)
        key = keys[group * dim:(group + 1) * dim]
        size = np.linalg.norm(key)
        set_column(bf16, "l0.mix.left.q", slice(head * dim, (head + 1) * dim), column,
                   14.0 / (size * 0.2 * h[probe][column]) * key / size)
    louder(bf16, "l0.mix.left.o", 8.0)
    return raw, bf16, changed, without


# (sizes, chunk, probe, far, seen): the first key of the probe's chunk and the last of the chunk before, with the
# probe as the last or the first position of a chunk, chunks of a page, of less, of no multiple of a page or tile,
# of several pages and tiles; a key 300 back without a mask; heads of the tensor-core kernels' sizes
EDGES = [((4, 2, 8, 12), 40, 119, 80, True), ((4, 2, 8, 12), 40, 119, 79, False), ((4, 2, 8, 12), 40, 120, 119, False),
         ((4, 2, 8, 12), 40, 121, 120, True), ((2, 1, 16, 16), 16, 63, 48, True), ((2, 1, 16, 16), 16, 63, 47, False),
         ((3, 3, 12, 5), 7, 300, 294, True), ((3, 3, 12, 5), 7, 300, 293, False), ((17, 1, 24, 8), 100, 299, 200, True),
         ((17, 1, 24, 8), 100, 299, 199, False), ((4, 2, 8, 12), None, 317, 0, True), ((4, 2, 8, 12), None, 317, 16, True),
         ((8, 2, 64, 64), 160, 319, 160, True), ((8, 2, 64, 64), 160, 319, 159, False), ((8, 1, 64, 128), 112, 340, 336, True),
         ((8, 1, 64, 128), 112, 340, 335, False), ((4, 4, 128, 64), 130, 389, 260, True), ((4, 4, 128, 64), 130, 389, 259, False),
         ((4, 2, 8, 12), 1, 50, 49, False), ((4, 2, 8, 12), 512, 317, 1, True)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes,chunk,probe,far,seen", EDGES)
def test_keys_just_inside_and_just_outside_a_chunk(tmp_path, sizes, chunk, probe, far, seen, dtype):
    """Whether the token at ``far`` is the one the probe's query points at moves the probe's logits if and only if
    both lie in one chunk; the engine follows the plain model with the probe inside a prompt, as the first token of
    a portion, in a portion that starts inside the chunk, and decoded alone (after a prompt and after decoded tokens)."""
    raw, bf16, changed, without = build_chunk_edge(sizes, chunk, probe, far, probe + 13)
    folder = str(tmp_path / "one")
    nm.write_model(folder, raw, 0, tensors=bf16)
    tensors = plain.as_float64(bf16)
    want, reference = plain.logits(raw, tensors, changed), plain.logits(raw, tensors, without)
    moved = spread_error(want[probe:probe + 1], reference[probe:probe + 1])[0]
    assert (moved > 0.2) if seen else (moved < 1e-9), f"the plain model itself: {moved}"
    loaded = load(folder, dtype)
    inside = max(far + 1, probe - 3) if far + 1 < probe else probe
    for tag, steps in (("prompt", [changed]), ("portion", [changed[:probe], changed[probe:]]),
                       ("inside", [changed[:inside], changed[inside:probe + 2], changed[probe + 2:]]),
                       ("decoded", [changed[:probe]] + [[t] for t in changed[probe:]]),
                       ("later", [changed[:max(far - 5, probe - 120, 1)]] + [[t] for t in changed[max(far - 5, probe - 120, 1):]])):
        got = run_steps(loaded, [[(tag, part)] for part in steps])[tag]
        check(got, want, dtype, f"chunk {chunk}, key at {far}, probe at {probe} {tag}")
        shown = spread_error(got[probe:probe + 1].astype(np.float64), reference[probe:probe + 1])[0]
        assert (shown > 0.15) if seen else (shown <= LIMIT[dtype]), f"{tag}: {shown}"
        loaded.step.end(tag)


def build_far_lightning(decay, far, probe, length):
    """One lightning layer: ONE token writes a large value under a key of its own (through an input dimension that
    only it has), ONE probe token's query points at that key (through another such dimension)."""
    raw = nm.single_layer(nm.lightning(2, 16, 24, decay))
    bf16 = nm.make_tensors(raw, 42)
    vocab, width = raw["vocab"], raw["width"]
    key_token, probe_token, other_token = vocab - 1, vocab - 2, vocab - 3
    key_column, probe_column = width - 2, width - 4
    single_out(bf16, key_token, key_column)
    single_out(bf16, probe_token, probe_column)
    changed = np.random.default_rng(10).integers(0, vocab - 3, size=length).tolist()
    for place in probe:
        changed[place] = probe_token
    without = list(changed)
    changed[far], without[far] = key_token, other_token
    h = normed_inputs(raw, bf16, changed)
    direction = np.zeros(16)
    direction[::2] = 6.0                                   # silu keeps large positive entries about as they are
    rng = np.random.default_rng(11)
    for head in range(2):
        set_column(bf16, "l0.mix.k", slice(16 * head, 16 * (head + 1)), key_column, direction / h[far][key_column])
        set_column(bf16, "l0.mix.q", slice(16 * head, 16 * (head + 1)), probe_column, direction / h[probe[0]][probe_column])
        set_column(bf16, "l0.mix.v", slice(24 * head, 24 * (head + 1)), key_column, 9.0 * rng.normal(size=24) / h[far][key_column])
    louder(bf16, "l0.mix.o", 8.0)
    return raw, bf16, changed, without


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_shows_through_the_lightning_state(tmp_path, dtype):
    """Whether the writing token stood at place 3 moves the logits 250 tokens later (decays close to one and one);
    the engine follows the plain model whether the tokens between came as one prompt, in portions, or one by one."""
    raw, bf16, changed, without = build_far_lightning([0.9990234375, 1.0], 3, [250, 255], 256)
    folder = str(tmp_path / "one")
    nm.write_model(folder, raw, 0, tensors=bf16)
    tensors = plain.as_float64(bf16)
    want, reference = plain.logits(raw, tensors, changed), plain.logits(raw, tensors, without)
    assert spread_error(want[[250, 255]], reference[[250, 255]]).min() > 0.2, "the plain model itself forgot the far token"
    loaded = load(folder, dtype)
    for tag, steps in (("whole", [changed]), ("portions", cut(changed, [2, 70, 33, 16, 7])),
                       ("decoded", [changed[:6]] + [[t] for t in changed[6:]])):
        got = run_steps(loaded, [[(tag, part)] for part in steps])[tag]
        check(got, want, dtype, f"lightning, {tag}")
        assert spread_error(got[[250, 255]].astype(np.float64), reference[[250, 255]]).min() > 0.15
        loaded.step.end(tag)


def build_far_recurrent(far, probe, length, taps=3):
    """One side-by-side layer whose left half counts for nothing. In the right half ONE token feeds a large input
    into channels that forget over hundreds of tokens (lam far below zero); the y branch of ONE probe token opens
    those channels wide."""
    raw = nm.single_layer(nm.parallel(1, 1, 4, 4, 5, 24, 2, taps, left_scale=0.0, right_scale=1.0))
    bf16 = nm.make_tensors(raw, 43)
    vocab, width = raw["vocab"], raw["width"]
    key_token, probe_token, other_token = vocab - 1, vocab - 2, vocab - 3
    key_column, probe_column = width - 2, width - 4
    single_out(bf16, key_token, key_column)
    single_out(bf16, probe_token, probe_column)
    changed = np.random.default_rng(12).integers(0, vocab - 3, size=length).tolist()
    for place in probe:
        changed[place] = probe_token
    without = list(changed)
    changed[far], without[far] = key_token, other_token
    h = normed_inputs(raw, bf16, changed)
    import torch
    lam = bf16["l0.mix.right.lam"].float().numpy().copy()
    lam[:12] = -7.0                                        # softplus about 1e-3: a = exp(-8 r 1e-3), half gone after ~170 tokens
    bf16["l0.mix.right.lam"] = torch.from_numpy(lam).to(torch.bfloat16)
    rng = np.random.default_rng(13)
    set_column(bf16, "l0.mix.right.x", slice(0, 12), key_column, 60.0 * rng.choice([-1.0, 1.0], size=12) / h[far][key_column])
    set_column(bf16, "l0.mix.right.y", slice(0, 12), probe_column, 5.0 / h[probe[0]][probe_column])
    louder(bf16, "l0.mix.right.o", 4.0)
    return raw, bf16, changed, without


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_shows_through_the_recurrent_unit(tmp_path, dtype):
    raw, bf16, changed, without = build_far_recurrent(3, [250, 255], 256)
    folder = str(tmp_path / "one")
    nm.write_model(folder, raw, 0, tensors=bf16)
    tensors = plain.as_float64(bf16)
    want, reference = plain.logits(raw, tensors, changed), plain.logits(raw, tensors, without)
    assert spread_error(want[[250, 255]], reference[[250, 255]]).min() > 0.2, "the plain model itself forgot the far token"
    loaded = load(folder, dtype)
    for tag, steps in (("whole", [changed]), ("portions", cut(changed, [2, 70, 33, 16, 7])),
                       ("decoded", [changed[:6]] + [[t] for t in changed[6:]])):
        got = run_steps(loaded, [[(tag, part)] for part in steps])[tag]
        check(got, want, dtype, f"recurrent unit, {tag}")
        assert spread_error(got[[250, 255]].astype(np.float64), reference[[250, 255]]).min() > 0.15
        loaded.step.end(tag)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("blocks,width", [(1, 16), (4, 40), (3, 132)])
def test_convolution_and_gates_across_portion_borders(tmp_path, taps, blocks, width):
    """Portions shorter than the convolution's reach, so that a token's inputs come from two and three portions
    back; the first tokens of a sequence meet zeros; parts of 16, 10 and 44 channels."""
    layer = nm.parallel(2, 1, 8, 8, 6, width, blocks, taps, left_scale=0.3, right_scale=1.2)
    folder, raw, tensors = one_layer_model(tmp_path, layer, 44 + taps)
    tokens = tokens_of(raw["vocab"], 61, 12)
    want = plain.logits(raw, tensors, tokens)
    loaded = load(folder, "float32")
    for tag, sizes in (("a", [1, 2, 2, 3, 1, 1, 5, 2]), ("b", [2]), ("c", [30, 1, 2, 28])):
        got = run_steps(loaded, [[(tag, part)] for part in cut(tokens, sizes)])[tag]
        check(got, want, "float32", f"{taps} taps, {blocks} blocks of {width // blocks}, portions of {sizes}")
        loaded.step.end(tag)


@pytest.mark.parametrize("dim,vdim", [(8, 5), (32, 32), (40, 70), (72, 16), (136, 24), (200, 8)])
def test_key_and_value_sizes_of_the_lightning_mixer(tmp_path, dim, vdim):
    """One, two, four and eight lanes a column, value sizes that fill no warp evenly; a decay of exactly one."""
    folder, raw, tensors = one_layer_model(tmp_path, nm.lightning(2, dim, vdim, [0.75, 1.0]), 44)
    tokens = tokens_of(raw["vocab"], 45, 12)
    want = plain.logits(raw, tensors, tokens)
    got = run_steps(load(folder, "float32"), [[("a", tokens[:20])], [("a", tokens[20:21])], [("a", tokens[21:])]])["a"]
    check(got, want, "float32", f"lightning with keys of {dim} and values of {vdim}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,shared", [(4, 1, None), (8, 8, 16), (40, 3, 24), (64, 6, None), (3, 2, 8)])
def test_experts_choices_and_the_shared_expert(tmp_path, experts, top, shared, dtype):
    """One layer whose feed-forward is a mixture: one choice, all experts chosen, more experts than a warp has
    lanes, with and without the shared expert; in steps of few tokens (the experts' rows stream) and of many
    (pairs grouped by expert), which must agree."""
    folder, raw, tensors = one_layer_model(tmp_path, nm.lightning(1, 8, 8), 45, mlp=nm.moe(experts, top, 24, shared=shared))
    tokens = tokens_of(raw["vocab"], 150, 13)
    want = plain.logits(raw, tensors, tokens)
    loaded = load(folder, dtype)
    whole = run_steps(loaded, [[("w", tokens)]])["w"]
    check(whole, want, dtype, f"{experts} experts, {top} chosen, whole", routed=True)
    pieces = run_steps(loaded, [[("p", part)] for part in cut(tokens, [3, 16, 17, 1, 40])])["p"]
    check(pieces, want, dtype, f"{experts} experts, {top} chosen, portions", routed=True)


def test_the_router_bias_moves_the_choice_and_the_weights(tmp_path):
    """A router bias that lifts two experts over all others: the engine chooses them and weighs them by the softmax
    of their lifted logits. Without it the output differs."""
    import torch
    raw = nm.single_layer(nm.lightning(1, 8, 8), nm.moe(6, 2, 16))
    bf16 = nm.make_tensors(raw, 46)
    tokens = tokens_of(raw["vocab"], 30, 14)
    outputs = []
    for tag, bias in (("plain", [0.0] * 6), ("lifted", [0.0, 40.0, 0.0, 0.0, 41.0, 0.0])):
        bf16["l0.mlp.router.b"] = torch.tensor(bias).to(torch.bfloat16)
        folder = str(tmp_path / tag)
        nm.write_model(folder, raw, 0, tensors=bf16)
        tensors = plain.as_float64(bf16)
        want = plain.logits(raw, tensors, tokens)
        check(run_steps(load(folder, "float32"), [[("a", tokens)]])["a"], want, "float32", f"router bias {tag}")
        outputs.append(want)
    tensors = plain.as_float64(bf16)
    streams = plain.embed(raw, tensors, tokens)
    eps = float(raw["norm"]["eps"])
    after_mixer = streams + plain.lightning(tensors, "l0.mix.", raw["layers"][0]["mixer"], plain.offset_norm(streams, tensors["l0.norm1"], eps), eps)
    chosen, weights = plain.route(tensors, "l0.mlp.", raw["layers"][0]["mlp"], plain.offset_norm(after_mixer, tensors["l0.norm2"], eps))
    assert set(np.unique(chosen)) == {1, 4}
    assert np.median(spread_error(outputs[0], outputs[1])) > 0.01


def test_the_first_tokens_of_a_sequence(tmp_path):
    """Prompts of one, two and three tokens and decoding from there: the convolution meets zeros, the recurrences
    start from zero with no special case, the first chunk holds one key."""
    for name, (raw, seed) in nm.CONFIGS.items():
        folder = str(tmp_path / name)
        raw, bf16 = nm.write_model(folder, raw, seed)
        tensors = plain.as_float64(bf16)
        tokens = tokens_of(raw["vocab"], 12, 16)
        want = plain.logits(raw, tensors, tokens)
        loaded = load(folder, "float32")
        for first in (1, 2, 3):
            got = run_steps(loaded, [[("f", tokens[:first])]] + [[("f", [t])] for t in tokens[first:]])["f"]
            check(got, want, "float32", f"{name}: a prompt of {first}")
            loaded.step.end("f")


# ---------------------------------------------------------------------------- the engine's own entry point
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_greedy_generation_through_the_engine(models, name):
    """Prompts of unequal length through ``Engine.generate`` (scheduler, portions, sampler) in float32 against
    greedy decoding with the plain model."""
    from celeg_b200 import Engine, EngineOptions
    folder, raw, tensors = models[name]
    prompts = [tokens_of(raw["vocab"], n, 50 + n) for n in (5, 41, 18)]
    new = 12
    engine = Engine(folder, max_context=128, dtype="float32",
                    options=EngineOptions(max_active_requests=4, max_batched_tokens=32, page_tokens=16))
    got = engine.generate(prompts, max_new_tokens=new, temperature=0.0, repetition_penalty=1.0)
    compared = 0
    for prompt, generated in zip(prompts, got):
        assert len(generated) == new
        sequence = list(prompt)
        for token in generated:
            logits = plain.logits(raw, tensors, sequence)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 1e-2 * (logits.max() - logits.min()):      # (no near tie in the plain model)
                assert int(token) == int(np.argmax(logits))
                compared += 1
            sequence.append(int(token))
    assert compared >= 2 * new


def test_greedy_generation_in_bfloat16_with_graphs(models):
    """The serving path (bfloat16, CUDA graphs, run-ahead): the tokens it generates are the plain model's wherever
    the plain model's best two logits are not close."""
    from celeg_b200 import Engine, EngineOptions
    folder, raw, tensors = models["mixed"]
    prompts = [tokens_of(raw["vocab"], n, 70 + n) for n in (9, 30)]
    engine = Engine(folder, max_context=128, dtype="bfloat16",
                    options=EngineOptions(max_active_requests=4, max_batched_tokens=64, page_tokens=16))
    got = engine.generate(prompts, max_new_tokens=10, temperature=0.0, repetition_penalty=1.0)
    for prompt, generated in zip(prompts, got):
        sequence = list(prompt)
        for token in generated:
            logits = plain.logits(raw, tensors, sequence)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 0.05 * (logits.max() - logits.min()):
                assert int(token) == int(np.argmax(logits))
            sequence.append(int(token))


def test_many_requests_through_a_small_pool(models):
    """Nine prompts through two slots and a pool of a few pages: the scheduler queues, admits as slots and pages
    come free, and every request's tokens are those of greedy decoding alone."""
    from celeg_b200 import Engine, EngineOptions
    folder, raw, tensors = models["odd"]
    prompts = [tokens_of(raw["vocab"], 3 + 5 * n, 200 + n) for n in range(9)]
    engine = Engine(folder, max_context=96, dtype="float32",
                    options=EngineOptions(max_active_requests=2, max_batched_tokens=24, page_tokens=16, logical_kv_pages=10))
    got = engine.generate(prompts, max_new_tokens=6, temperature=0.0, repetition_penalty=1.0)
    for prompt, generated in zip(prompts, got):
        sequence = list(prompt)
        for token in generated:
            logits = plain.logits(raw, tensors, sequence)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 1e-2 * (logits.max() - logits.min()):
                assert int(token) == int(np.argmax(logits))
            sequence.append(int(token))


def test_command_line_generates_and_dumps_logits(models, tmp_path, capsys):
    from celeg_b200.cli import main
    folder, raw, tensors = models["odd"]
    prompt = tokens_of(raw["vocab"], 12, 90)
    dump = str(tmp_path / "last.f32")
    code = main(["--model", folder, "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", "fp32",
                 "--temperature", "0", "--repetition-penalty", "1.0", "--runtime-tokens", "--dump-logits", dump,
                 "--context", "128"])
    assert code == 0
    captured = capsys.readouterr()
    sequence = list(prompt)
    for _ in range(6):
        sequence.append(int(np.argmax(plain.logits(raw, tensors, sequence)[-1])))
    assert f"CELEG_GENERATED_TOKEN_IDS=[{','.join(map(str, sequence[len(prompt):]))}]" in captured.out
    logits = np.fromfile(dump, dtype="<f4").astype(np.float64)
    assert spread_error(logits[None, :], plain.logits(raw, tensors, prompt)[-1:])[0] < 2e-4
    assert main(["--model", folder, "--print-config"]) == 0
    assert '"architecture": "Naselorn"' in capsys.readouterr().out


# ------------------------------------------------------------------------------- configurations drawn at random
def random_config(rng):
    width = int(rng.choice([20, 36, 64, 100, 128]))
    vocab = int(rng.integers(17, 300))
    layers = []
    for _ in range(int(rng.integers(1, 6))):
        if rng.random() < 0.5:
            heads, groups = [(1, 1), (2, 1), (4, 2), (6, 2), (8, 8), (12, 3), (20, 1)][int(rng.integers(0, 7))]
            dim = int(rng.choice([4, 8, 12, 32, 64]))
            vdim = int(rng.choice([4, 9, 16, 64, 128]))
            blocks = int(rng.choice([1, 2, 3, 8]))
            layer = nm.parallel(heads, groups, dim, vdim, None if rng.random() < 0.2 else int(rng.choice([1, 3, 16, 33, 64, 100])),
                                blocks * int(rng.choice([1, 5, 16, 40])), blocks, int(rng.integers(1, 6)),
                                scale=float(rng.choice([dim ** -0.5, 0.125, 0.5])),
                                left_scale=float(rng.choice([1.0, 0.7, 1.2])), right_scale=float(rng.choice([1.0, 0.9, -0.5])))
        else:
            heads = int(rng.integers(1, 5))
            layer = nm.lightning(heads, int(rng.choice([4, 8, 20, 32, 64, 130])), int(rng.choice([4, 9, 32, 80])),
                                 [float(rng.choice([0.5, 0.9, 0.96875, 0.999, 1.0])) for _ in range(heads)])
        pick = rng.random()
        if pick < 0.2:
            mlp = None
        elif pick < 0.55:
            mlp = nm.dense(int(rng.choice([8, 44, 128])))
        else:
            experts = int(rng.choice([2, 3, 8, 16, 33, 70]))
            mlp = nm.moe(experts, int(rng.integers(1, min(experts, 8) + 1)), int(rng.choice([8, 20, 64])),
                         shared=None if rng.random() < 0.4 else int(rng.choice([8, 36])))
        layers.append(nm.with_mlp(layer, mlp))
    return nm.config(vocab, width, layers, eps=float(rng.choice([1e-5, 1e-6, 1e-3])),
                     scale=float(rng.choice([1.0, width ** 0.5, 3.0])))


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Whole prompt, portions beside single tokens of a second request, and decoding, in both precisions."""
    rng = np.random.default_rng(3000 + seed)
    raw = random_config(rng)
    folder = str(tmp_path / "drawn")
    raw, bf16 = nm.write_model(folder, raw, 700 + seed)
    tensors = plain.as_float64(bf16)
    first, second = tokens_of(raw["vocab"], 75, seed), tokens_of(raw["vocab"], 33, 100 + seed)
    want = {"a": plain.logits(raw, tensors, first), "b": plain.logits(raw, tensors, second)}
    steps = [[("a", first[:19])], [("a", first[19:21]), ("b", second[:1])], [("b", second[1:2]), ("a", first[21:60])],
             [("a", first[60:61]), ("b", second[2:30])]]
    steps += [[("a", first[61 + i:62 + i])] + ([("b", second[30 + i:31 + i])] if 30 + i < len(second) else []) for i in range(14)]
    for dtype in ("float32", "bfloat16"):
        loaded = load(folder, dtype, page_tokens=int(rng.choice([8, 16, 32])))
        whole = run_steps(loaded, [[("w", first)]])["w"]
        loaded.step.end("w")
        got = run_steps(loaded, steps)
        if dtype == "float32":
            check(whole, want["a"], dtype, f"{raw['layers']} whole")
            for key in ("a", "b"):
                check(got[key], want[key], dtype, f"{raw['layers']} request {key}")
        else:
            for rows, target in ((whole, want["a"]), (got["a"], want["a"]), (got["b"], want["b"])):
                assert np.median(spread_error(np.asarray(rows, dtype=np.float64), target)) < 0.1


# ------------------------------------------------------------------------------------------ trace replay
def replay_steps(requests, seed):
    """A schedule for up to four live requests: portions of changing size (two tokens too) beside single tokens,
    requests left out of steps, ended requests followed by new ones. Returns (steps, {request: wanted places})."""
    rng = np.random.default_rng(seed)
    waiting = list(requests)
    live, at, steps = [], {}, []
    while waiting or live:
        while waiting and len(live) < 4:
            name = waiting.pop(0)
            live.append(name)
            at[name] = 0
        entries, ended = [], []
        for name in list(live):
            tokens = requests[name]
            left = len(tokens) - at[name]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                       # (left out of this step)
            count = min(left, int(rng.choice([1, 1, 2, 3, 17, 40])))
            entries.append({"id": name, "tokens": tokens[at[name]:at[name] + count], "want": list(range(count))})
            at[name] += count
            if at[name] == len(tokens):
                ended.append(name)
                live.remove(name)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


LIGHTNING_ONLY = nm.config(70, 40, [nm.with_mlp(nm.lightning(2, 8, 12, [0.9, 1.0]), nm.dense(24)),
                                    nm.with_mlp(nm.lightning(1, 20, 4), None)])
PARALLEL_ONLY = nm.config(90, 24, [nm.with_mlp(nm.parallel(2, 2, 8, 4, 9, 16, 2, 3), None),
                                   nm.with_mlp(nm.parallel(4, 1, 4, 8, None, 8, 1, 2, scale=0.4), nm.moe(3, 2, 8))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "lightning_only", "parallel_only"])
def test_replay_with_pages_and_slots_used_again(models, name, dtype, tmp_path):
    """Seven requests (640 positions in whole blocks of 64) through the trace runner's step loop with a pool for 448
    positions, what four live ones can hold at most, and four slots."""
    import io
    import json
    import os
    from celeg_b200.engine.trace import replay
    if name in models:
        folder, raw, tensors = models[name]
    else:
        folder = str(tmp_path / name)
        raw, bf16 = nm.write_model(folder, LIGHTNING_ONLY if name == "lightning_only" else PARALLEL_ONLY, 77)
        tensors = plain.as_float64(bf16)
    lengths = [70, 9, 100, 33, 64, 2, 81]
    requests = {f"r{i}": tokens_of(raw["vocab"], n, 300 + i) for i, n in enumerate(lengths)}
    steps = replay_steps(requests, 5)
    out_dir = str(tmp_path / f"out_{dtype}")
    done = io.StringIO()
    text = io.StringIO("".join(json.dumps(step) + "\n" for step in steps))
    assert replay(folder, dtype, out_dir, 448, text, done, max_requests=4) == 0
    assert done.getvalue().split() == [w for step in steps for w in ("done", str(step["step"]))]
    rows = {key: [] for key in requests}
    for step in steps:
        data = np.fromfile(os.path.join(out_dir, f"{step['step']}.f32"), dtype="<f4").reshape(-1, raw["vocab"])
        row = 0
        for entry in step["entries"]:
            rows[entry["id"]].append(data[row:row + len(entry["want"])])
            row += len(entry["want"])
        assert row == data.shape[0]
    for key, tokens in requests.items():
        check(np.concatenate(rows[key]), plain.logits(raw, tensors, tokens), dtype, f"{name} request {key} replayed", routed=True)


def test_the_trace_runner_as_a_program(models, tmp_path):
    import json
    import os
    import subprocess
    import sys
    folder, raw, tensors = models["odd"]
    tokens = tokens_of(raw["vocab"], 21, 400)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:18], "want": [0, 17]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[18:20], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[20:], "want": [0]}], "end": ["a"]}]
    program = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    out_dir = str(tmp_path / "out")
    result = subprocess.run([program, "--model", folder, "--dtype", "float32", "--out", out_dir, "--max-tokens", "64"],
                            input="".join(json.dumps(step) + "\n" for step in steps), capture_output=True, text=True,
                            timeout=600, env=dict(os.environ, PYTHON=sys.executable))
    assert result.returncode == 0, result.stderr[-2000:]
    assert [line for line in result.stdout.split("\n") if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out_dir, "1.f32"))
    want = plain.logits(raw, tensors, tokens)
    got = np.concatenate([np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4").reshape(-1, raw["vocab"]) for n in (0, 2)])
    check(got, want[[0, 17, 20]], "float32", "the program's logits")


# ------------------------------------------------------------------------------- layers of a real model's size
@pytest.fixture(scope="module")
def large(tmp_path_factory):
    """Three layers 1,024 wide: lightning heads of 64 keys and 128 values with 32 gated experts and a shared one; eight
    attention heads of 128 on two key heads under chunks of 256 beside a recurrent unit of 1,024 channels in blocks of
    128 behind four taps, with a ReLU-gated feed-forward; lightning again. The sizes at which the grouped tensor-core
    product, the segmented scan, the tensor-core attention kernels and the wide row norm are the ones that run."""
    decay = [1.0 - 2.0 ** (-3 - head) for head in range(8)]
    raw = nm.config(8192, 1024, [
        nm.with_mlp(nm.lightning(8, 64, 128, decay), nm.moe(32, 4, 512, shared=1024)),
        nm.with_mlp(nm.parallel(8, 2, 128, 128, 256, 1024, 8, 4, left_scale=1.1, right_scale=0.8), nm.dense(2816)),
        nm.with_mlp(nm.lightning(8, 64, 128, decay), nm.dense(1536)),
    ])
    folder = str(tmp_path_factory.mktemp("naselorn_large") / "model")
    raw, bf16 = nm.write_model(folder, raw, 91)
    tensors = plain.as_float64(bf16)
    first, second = tokens_of(raw["vocab"], 608, 500), tokens_of(raw["vocab"], 450, 501)
    return folder, raw, {"a": first, "b": second}, {"a": plain.logits(raw, tensors, first), "b": plain.logits(raw, tensors, second)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_a_real_model_size(large, dtype):
    folder, raw, requests, want = large
    first, second = requests["a"], requests["b"]
    loaded = load(folder, dtype, cache_tokens=2048, max_batched_tokens=1024, max_context=1024)
    steps = [[("a", first[:600])], [("a", first[600:601]), ("b", second[:300])], [("a", first[601:602]), ("b", second[300:])]]
    steps += [[("a", [t])] for t in first[602:]]
    got = run_steps(loaded, steps)
    for key in ("a", "b"):
        check(got[key], want[key], dtype, f"request {key} at a real model's layer sizes", routed=True)
