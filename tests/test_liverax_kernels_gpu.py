"""The kernels that the Liverax design added or widened, each against the same operation written in numpy (float64):
the layer norm with the residual add, the strided RMS norm, the sigmoid gate, the preparation of q, k and v (biases,
whole-projection norms, rotation of halves, the query factor, value blending, the cache write), score biases by
distance in all four attention kernels (also with a table that lets exactly one distance through), the latent
preparation with pairs of halves, and the per-head product with a gate per element."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"


def kernels():
    from celeg_b200 import kernels as k
    return k


def gpu(array, dtype=torch.float32):
    return torch.as_tensor(np.asarray(array)).to(dtype).to(DEVICE).contiguous()


def close(got: torch.Tensor, want: np.ndarray, rel: float, what: str):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    scale = np.abs(want).max() + 1e-30
    worst = np.abs(got - want).max() / scale
    assert worst <= rel, f"{what}: differs by {worst:.3e} of the largest value"


def bf16_round(array):
    return torch.as_tensor(np.asarray(array, dtype=np.float32)).to(torch.bfloat16).to(torch.float64).numpy()


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


# ------------------------------------------------------------------------------------------------- norms
@pytest.mark.parametrize("dtype,rel", [(torch.float32, 3e-6), (torch.bfloat16, 6e-3)])
@pytest.mark.parametrize("rows,width", [(5, 36), (3, 64), (7, 515), (2, 4096), (2, 8192), (3, 9000)])
def test_layer_norm_adds_centres_and_scales(rows, width, dtype, rel):
    k = kernels()
    rng = np.random.default_rng(width)
    residual = rng.normal(5.0, 2.0, size=(rows, width))          # a mean that is large beside the spread
    delta = bf16_round(rng.normal(size=(rows, width))) if dtype == torch.bfloat16 else rng.normal(size=(rows, width))
    weight, bias = rng.normal(1.0, 0.3, size=width), rng.normal(size=width)
    eps = 1e-5

    def plain(x, b=None):
        centred = x - x.mean(-1, keepdims=True)
        out = centred / np.sqrt((centred ** 2).mean(-1, keepdims=True) + eps) * weight
        return out if b is None else out + b
    stream = gpu(residual)
    out = torch.zeros((rows, width), dtype=dtype, device=DEVICE)
    k.add_layernorm(stream, gpu(delta, dtype), gpu(weight), out, eps, n_rows=rows)
    x = residual.astype(np.float32).astype(np.float64) + delta
    close(out, plain(x), rel, "layer norm with the add")
    close(stream, x, 1e-6, "the stream after the add")
    k.add_layernorm(stream, None, gpu(weight), out, eps, n_rows=rows, bias=gpu(bias))
    close(out, plain(x, bias), rel, "layer norm with a bias, nothing to add")
    picked = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEVICE)
    before = stream.clone()
    k.add_layernorm(stream, gpu(delta, dtype), gpu(weight), out, eps, rows=picked, n_rows=2)
    close(out[:2], plain(x + delta)[[rows - 1, 0]], rel, "layer norm of gathered rows")
    assert torch.equal(stream, before)                            # (a gathered norm leaves the stream alone)


@pytest.mark.parametrize("dtype,rel", [(torch.float32, 3e-6), (torch.bfloat16, 6e-3)])
def test_rms_norm_of_a_slice_and_the_sigmoid_gate(dtype, rel):
    k = kernels()
    rng = np.random.default_rng(3)
    rows, width, offset, total = 6, 40, 8, 100
    wide = bf16_round(rng.normal(size=(rows, total)) * 3) if dtype == torch.bfloat16 else rng.normal(size=(rows, total)) * 3
    weight = rng.normal(1.0, 0.3, size=width)
    x = wide[:, offset:offset + width]
    want = x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-4) * weight
    out = torch.zeros((rows, width + 4), dtype=dtype, device=DEVICE)
    k.rmsnorm_strided(gpu(wide, dtype)[:, offset:offset + width], gpu(weight), out[:, :width], 1e-4, rows)
    close(out[:, :width], want, rel, "RMS norm of a slice")
    values = bf16_round(rng.normal(size=(rows, width))) if dtype == torch.bfloat16 else rng.normal(size=(rows, width))
    for gate_type in {torch.float32, dtype}:
        held = gpu(values, dtype)
        gate = bf16_round(wide) if gate_type == torch.bfloat16 else wide
        k.sigmoid_gate(held, gpu(gate, gate_type)[:, offset:offset + width], rows, width)
        close(held, values * sigmoid(gate[:, offset:offset + width]), rel, f"sigmoid gate from {gate_type}")


# --------------------------------------------------------------------------------------- the paged cache
class Paged:
    """Spans of (positions already cached, new tokens) over pages handed out in a scrambled order."""

    def __init__(self, spans, kv_heads, head_dim, value_dim, page_tokens, dtype, seed):
        rng = np.random.default_rng(seed)
        self.spans, self.page_tokens = spans, page_tokens
        needed = [-(-(before + new) // page_tokens) for before, new in spans]
        pages = sum(needed) + 3
        order = rng.permutation(pages)
        self.table = np.full((len(spans), max(needed) + 1), -1, dtype=np.int32)
        at = 0
        for s, n in enumerate(needed):
            self.table[s, :n] = order[at:at + n]
            at += n
        self.positions = np.concatenate([np.arange(before, before + new) for before, new in spans]).astype(np.int32)
        self.token_span = np.concatenate([np.full(new, s) for s, (_, new) in enumerate(spans)]).astype(np.int32)
        self.span_begin = np.concatenate([[0], np.cumsum([new for _, new in spans])]).astype(np.int32)
        self.tokens = int(self.span_begin[-1])
        self.k = torch.zeros((pages, kv_heads, page_tokens, head_dim), dtype=dtype, device=DEVICE)
        self.v = torch.zeros((pages, kv_heads, page_tokens, value_dim), dtype=dtype, device=DEVICE)
        self.flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)

    def fill(self, keys, values):
        """keys[s]: [before + new, kv_heads, head_dim] of span s (values alike) into its pages."""
        for s, (before, new) in enumerate(self.spans):
            for pos in range(before + new):
                page, place = self.table[s, pos // self.page_tokens], pos % self.page_tokens
                self.k[page, :, place] = gpu(keys[s][pos], self.k.dtype)
                self.v[page, :, place] = gpu(values[s][pos], self.v.dtype)

    def read(self, cache, s, pos):
        return cache[self.table[s, pos // self.page_tokens], :, pos % self.page_tokens].float().cpu().numpy().astype(np.float64)

    def device(self):
        return (gpu(self.positions, torch.int32), gpu(self.token_span, torch.int32), gpu(self.span_begin, torch.int32),
                gpu(self.table, torch.int32))


# ------------------------------------------------------------------------------- preparation of q, k and v
@pytest.mark.parametrize("dtype,rel", [(torch.float32, 3e-6), (torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("heads,groups,dim,vdim,key_store,value_store,rotary,norms,temp,blend",
                         [(4, 2, 16, 16, 16, 16, 8, False, None, 1), (3, 1, 12, 7, 12, 7, 12, True, (0.5, 3), 2),
                          (2, 2, 64, 32, 64, 64, 0, True, (0.25, 10), 0), (8, 1, 128, 128, 128, 128, 64, False, None, 2),
                          (5, 5, 6, 6, 8, 8, 2, True, None, 0)])
def test_preparation_of_queries_keys_and_values(heads, groups, dim, vdim, key_store, value_store, rotary, norms, temp,
                                                blend, dtype, rel):
    k = kernels()
    rng = np.random.default_rng(heads * 100 + dim)
    spans = [(0, 5), (37, 1), (14, 9)]
    paged = Paged(spans, groups, key_store, value_store, 16, dtype, 1)
    tokens = paged.tokens
    qw, kw, vw = heads * dim, groups * dim, groups * vdim
    proj = rng.normal(size=(tokens, qw + kw + vw + 5))                    # (rows wider than q | k | v)
    bias = rng.normal(size=qw + kw + vw)
    q_norm, k_norm = rng.normal(1.0, 0.3, size=qw), rng.normal(1.0, 0.3, size=kw)
    frequencies = (50.0 ** (-2.0 * np.arange(rotary // 2) / max(rotary, 1)) / 1.5).astype(np.float32)
    first = rng.normal(size=(tokens, vw)).astype(np.float32)
    lam, eps = 0.3, 1e-5
    positions, token_span, _, table = paged.device()
    q_out = torch.zeros((tokens, heads * key_store), dtype=dtype, device=DEVICE)
    first_dev = gpu(first)
    k.qkv_prepare(gpu(proj), gpu(bias), q_out, positions, token_span, table, paged.k, paged.v, tokens, heads, groups, dim,
                  vdim, key_store, value_store, 16, paged.flag, q_norm=gpu(q_norm) if norms else None,
                  k_norm=gpu(k_norm) if norms else None, norm_eps=eps, frequencies=gpu(frequencies) if rotary else None,
                  rotary_dim=rotary, temperature=temp, blend=blend, lam=lam, first_values=first_dev if blend else None)
    assert int(paged.flag.item()) == 0
    x = proj.astype(np.float32).astype(np.float64)[:, :qw + kw + vw] + bias.astype(np.float32)
    q, kk, v = x[:, :qw], x[:, qw:qw + kw], x[:, qw + kw:]
    if norms:
        q = q / np.sqrt((q ** 2).mean(-1, keepdims=True) + eps) * q_norm.astype(np.float32)
        kk = kk / np.sqrt((kk ** 2).mean(-1, keepdims=True) + eps) * k_norm.astype(np.float32)
    q, kk = q.reshape(tokens, heads, dim).copy(), kk.reshape(tokens, groups, dim).copy()
    half = rotary // 2
    for rows in (q, kk):
        if rotary:
            angles = paged.positions[:, None].astype(np.float64) * frequencies[None, :].astype(np.float64)
            cos, sin = np.cos(angles)[:, None, :], np.sin(angles)[:, None, :]
            a, b = rows[..., :half].copy(), rows[..., half:rotary].copy()
            rows[..., :half], rows[..., half:rotary] = a * cos - b * sin, b * cos + a * sin
    if temp:
        q = q * (1.0 + temp[0] * np.log((paged.positions + 1) // temp[1] + 1.0))[:, None, None]
    if blend == 2:
        v = (1.0 - lam) * v + lam * first
    got_q = q_out.float().cpu().numpy().reshape(tokens, heads, key_store)
    close(torch.as_tensor(got_q[..., :dim]), q, rel, "queries")
    assert not got_q[..., dim:].any()
    if blend == 1:
        close(first_dev, v, 1e-6, "the values noted for later layers")
    for t in range(tokens):
        s, pos = int(paged.token_span[t]), int(paged.positions[t])
        stored_k, stored_v = paged.read(paged.k, s, pos), paged.read(paged.v, s, pos)
        close(torch.as_tensor(stored_k[:, :dim]), kk[t], rel, f"the key of token {t}")
        close(torch.as_tensor(stored_v[:, :vdim]), v[t].reshape(groups, vdim), rel, f"the value of token {t}")
        assert not stored_k[:, dim:].any() and not stored_v[:, vdim:].any()


# ------------------------------------------------------------------------------- score biases by distance
def plain_attention(queries, keys, values, spans, scale, window, bias, sinks):
    """queries[t]: [heads, dim] of the new tokens in order; keys[s] / values[s]: [positions, groups, dim]; bias:
    [heads, last + 1] or None. Returns [tokens, heads, vdim]."""
    heads = queries.shape[1]
    group = heads // keys[0].shape[1]
    out, t = [], 0
    for s, (before, new) in enumerate(spans):
        for pos in range(before, before + new):
            first = 0 if not window else max(0, pos - window + 1)
            row = np.zeros((heads, values[s].shape[2]))
            for h in range(heads):
                scores = keys[s][first:pos + 1, h // group] @ queries[t, h] * scale
                if bias is not None:
                    back = pos - np.arange(first, pos + 1)
                    scores = scores + bias[h, np.minimum(back, bias.shape[1] - 1)]
                top = scores.max() if sinks is None else max(scores.max(), sinks[h])
                e = np.exp(scores - top)
                denominator = e.sum() + (0.0 if sinks is None else math.exp(sinks[h] - top))
                row[h] = (e / denominator) @ values[s][first:pos + 1, h // group]
            out.append(row)
            t += 1
    return np.stack(out)


def attention_case(heads, groups, dim, spans, last, seed, one_distance=None):
    rng = np.random.default_rng(seed)
    tokens = sum(new for _, new in spans)
    queries = bf16_round(rng.normal(size=(tokens, heads, dim)))
    keys = [bf16_round(rng.normal(size=(before + new, groups, dim))) for before, new in spans]
    values = [bf16_round(rng.normal(size=(before + new, groups, dim))) for before, new in spans]
    bias = rng.normal(0.0, 2.0, size=(heads, last + 1)).astype(np.float32).astype(np.float64)
    if one_distance is not None:
        # nothing in q: every score is its bias, and one distance stands forty above all others
        queries = np.zeros_like(queries)
        bias = np.zeros((heads, last + 1))
        bias[:, one_distance] = 40.0
    return queries, keys, values, bias


KERNELS = ["generic", "prefill", "tcgen05", "decode"]


def run_attention(kind, paged, queries, heads, groups, dim, scale, window, bias, sinks, dtype):
    k = kernels()
    positions, token_span, span_begin, table = paged.device()
    tokens = paged.tokens
    q = gpu(queries.reshape(tokens, heads * dim), dtype)
    out = torch.zeros((tokens, heads * dim), dtype=dtype, device=DEVICE)
    bias_dev = gpu(bias) if bias is not None else None
    sinks_dev = gpu(sinks) if sinks is not None else None
    spans = len(paged.spans)
    if kind == "generic":
        k.attention_generic(q, heads * dim, out, paged.k, paged.v, positions, token_span, table, tokens, heads, groups, dim,
                            paged.page_tokens, window, scale, paged.flag, sinks=sinks_dev, distance_bias=bias_dev)
    elif kind == "prefill":
        k.attention_prefill(q, heads * dim, out, paged.k, paged.v, positions, span_begin, table, tokens, spans, heads,
                            groups, dim, paged.page_tokens, window, scale, paged.flag, sinks=sinks_dev, distance_bias=bias_dev)
    elif kind == "tcgen05":
        tiles = sum(-(-new // 128) for _, new in paged.spans)
        k.attention_prefill_tcgen05(q, heads * dim, out, paged.k, paged.v, positions, span_begin, table, tokens, spans,
                                    tiles, heads, groups, dim, paged.page_tokens, window, scale, paged.flag,
                                    sinks=sinks_dev, distance_bias=bias_dev)
    else:
        chunk, splits = 128, 8
        partial_o = torch.zeros(tokens * heads * splits * dim, dtype=torch.float32, device=DEVICE)
        partial_ml = torch.zeros(tokens * heads * splits * 2, dtype=torch.float32, device=DEVICE)
        counters = torch.zeros(tokens * groups, dtype=torch.int32, device=DEVICE)
        k.attention_decode(q, heads * dim, out, paged.k, paged.v, positions, token_span, table, tokens, heads, groups, dim,
                           paged.page_tokens, window, scale, chunk, splits, partial_o, partial_ml, counters, paged.flag,
                           sinks=sinks_dev, distance_bias=bias_dev)
    torch.cuda.synchronize()
    assert int(paged.flag.item()) == 0
    return out.float().cpu().numpy().reshape(tokens, heads, dim).astype(np.float64)


@pytest.mark.parametrize("kind", KERNELS)
@pytest.mark.parametrize("heads,groups,dim,window,last,with_sinks", [(4, 2, 64, None, 100, False), (2, 1, 64, 70, 30, True),
                                                                    (8, 1, 128, None, 300, False), (3, 3, 24, None, 9, True)])
def test_score_biases_by_distance_in_every_attention_kernel(kind, heads, groups, dim, window, last, with_sinks):
    if kind == "tcgen05" and dim != 64:
        pytest.skip("the tcgen05 kernel takes heads of 64")
    decoding = kind == "decode"
    spans = [(450, 1), (0, 1), (129, 1), (63, 1)] if decoding else [(0, 200), (310, 3), (100, 129), (5, 1)]
    queries, keys, values, bias = attention_case(heads, groups, dim, spans, last, dim + heads)
    sinks = np.linspace(-1.0, 2.0, heads) if with_sinks else None
    scale = 0.7 / math.sqrt(dim)
    want = plain_attention(queries, keys, values, spans, scale, window, bias, sinks)
    for dtype, rel in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        if dtype == torch.float32 and kind != "generic":
            continue
        paged = Paged(spans, groups, dim, dim, 16, dtype, 2)
        paged.fill(keys, values)
        got = run_attention(kind, paged, queries, heads, groups, dim, scale, window, bias, sinks, dtype)
        close(torch.as_tensor(got), want, rel, f"{kind} attention with biases by distance")


@pytest.mark.parametrize("kind", KERNELS)
@pytest.mark.parametrize("distance,last", [(0, 40), (1, 40), (17, 40), (39, 40), (40, 40), (64, 200), (127, 200), (128, 200)])
def test_exactly_one_distance_gets_through(kind, distance, last):
    """No query, a table that is zero but for one distance: every token's result is the value that many positions
    back (for the table's last entry: the mean over everything that far and farther, which shares it)."""
    heads, groups, dim = 4, 2, 64
    decoding = kind == "decode"
    spans = [(300, 1), (distance, 1), (130, 1)] if decoding else [(0, 140), (250, 40), (distance, 2)]
    queries, keys, values, bias = attention_case(heads, groups, dim, spans, last, 7, one_distance=distance)
    want = plain_attention(queries, keys, values, spans, 1.0, None, bias, None)
    if distance < last:                                   # (the plain sum itself picks one value)
        t = 0
        for s, (before, new) in enumerate(spans):
            for pos in range(before, before + new):
                if pos >= distance:
                    assert np.allclose(want[t, 0], values[s][pos - distance, 0], atol=1e-6)
                t += 1
    dtype = torch.float32 if kind == "generic" else torch.bfloat16
    paged = Paged(spans, groups, dim, dim, 16, dtype, 3)
    paged.fill(keys, values)
    got = run_attention(kind, paged, queries, heads, groups, dim, 1.0, None, bias, None, dtype)
    close(torch.as_tensor(got), want, 1e-5 if dtype == torch.float32 else 1e-2, f"{kind}: distance {distance} alone")


# ----------------------------------------------------------------------------------- the latent mixer's kernels
@pytest.mark.parametrize("dtype,rel", [(torch.float32, 3e-6), (torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("halves", [False, True])
def test_latent_preparation_pairs_neighbours_or_halves(halves, dtype, rel):
    k = kernels()
    rng = np.random.default_rng(5)
    heads, dim, rot, rotated, rank = 3, 8, 12, 8, 20
    spans = [(9, 4), (0, 2)]
    paged = Paged(spans, 1, rank + rot, 1, 16, dtype, 4)
    tokens = paged.tokens
    rounded = bf16_round if dtype == torch.bfloat16 else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    q, down = rounded(rng.normal(size=(tokens, heads * (dim + rot)))), rounded(rng.normal(size=(tokens, rank + rot)))
    weight = rng.normal(1.0, 0.3, size=rank).astype(np.float32)
    frequencies = (100.0 ** (-2.0 * np.arange(rotated // 2) / rotated)).astype(np.float32)
    positions, token_span, _, table = paged.device()
    query = torch.zeros((tokens, heads * (rank + rot)), dtype=dtype, device=DEVICE)
    cache = paged.k.view(paged.k.shape[0], 16, rank + rot)
    k.latent_prepare(gpu(q, dtype), gpu(down, dtype), gpu(weight), gpu(frequencies), 1.0, 1e-5, positions, token_span, table,
                     cache, 16, query, tokens, heads, dim, rot, rotated, rank, paged.flag, halves=halves)
    half = rotated // 2
    pairs = [(i, i + half) for i in range(half)] if halves else [(2 * i, 2 * i + 1) for i in range(half)]

    def turn(part, position):
        out = part.copy()
        for i, (a, b) in enumerate(pairs):
            angle = float(np.float32(position) * frequencies[i])
            out[..., a] = part[..., a] * math.cos(angle) - part[..., b] * math.sin(angle)
            out[..., b] = part[..., b] * math.cos(angle) + part[..., a] * math.sin(angle)
        return out
    got_query = query.float().cpu().numpy().reshape(tokens, heads, rank + rot)
    for t in range(tokens):
        s, pos = int(paged.token_span[t]), int(paged.positions[t])
        c = down[t, :rank] / math.sqrt((down[t, :rank] ** 2).mean() + 1e-5) * weight
        stored = paged.read(paged.k, s, pos)[0]
        close(torch.as_tensor(stored[:rank]), c, rel, "the latent vector")
        close(torch.as_tensor(stored[rank:]), turn(down[t, rank:], pos), rel, "the shared key part")
        want_q = turn(q[t].reshape(heads, dim + rot)[:, dim:], pos)
        close(torch.as_tensor(got_query[t, :, rank:]), want_q, rel, "the queries' rotated parts")


@pytest.mark.parametrize("dtype,rel", [(torch.float32, 3e-6), (torch.bfloat16, 8e-3)])
def test_per_head_product_with_a_gate_per_element(dtype, rel):
    k = kernels()
    rng = np.random.default_rng(6)
    tokens, heads, n, kk = 70, 3, 20, 24
    rounded = bf16_round if dtype == torch.bfloat16 else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    x, matrix = rounded(rng.normal(size=(tokens, heads * (kk + 4)))), rounded(rng.normal(size=(heads * n, kk)) / 5)
    gate = rounded(rng.normal(size=(tokens, heads * n)))
    out = torch.zeros((tokens, heads * n), dtype=dtype, device=DEVICE)
    k.head_project(gpu(x, dtype), kk + 4, gpu(matrix, dtype), False, out, n, tokens, heads, n, kk, gate=gpu(gate, dtype),
                   gate_per_element=True)
    read = x.reshape(tokens, heads, kk + 4)[:, :, :kk]
    want = np.einsum("thk,hnk->thn", read, matrix.reshape(heads, n, kk)).reshape(tokens, heads * n) * sigmoid(gate)
    close(out, want, rel, "per-head product with a gate per element")
    per_head = rounded(rng.normal(size=(tokens, heads)))
    k.head_project(gpu(x, dtype), kk + 4, gpu(matrix, dtype), False, out, n, tokens, heads, n, kk, gate=gpu(per_head, dtype))
    want = np.einsum("thk,hnk->thn", read, matrix.reshape(heads, n, kk)) * sigmoid(per_head)[:, :, None]
    close(out, want.reshape(tokens, heads * n), rel, "per-head product with a gate per head")


# ------------------------------------------------------------------- the gated product on the tcgen05 tensor cores
@pytest.mark.parametrize("variant", [-1, 1, 3])
@pytest.mark.parametrize("rows,k,inner", [(300, 64, 128), (700, 256, 384), (129, 72, 40)])
def test_gated_product_with_another_gate_function_on_tcgen05(rows, k, inner, variant):
    """[gate | up] in one tcgen05 product with the tanh form of GELU, and with ReLU, on the gate in the epilogue; SiLU
    through the same code still gives what the SwiGLU epilogue gave."""
    kn = kernels()
    rng = np.random.default_rng(rows + k)
    x = torch.as_tensor(rng.normal(size=(rows, k)), dtype=torch.float32).to(torch.bfloat16).to(DEVICE)
    w = torch.as_tensor(rng.normal(size=(2 * inner, k)) / math.sqrt(k), dtype=torch.float32).to(torch.bfloat16).to(DEVICE)
    flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    ref = x.double() @ w.double().t()
    g = ref[:, :inner].to(torch.bfloat16).double()
    u = ref[:, inner:].to(torch.bfloat16).double()
    gates = {kn.ACT_GELU_TANH: 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))),
             kn.ACT_RELU: torch.clamp(g, min=0.0), kn.ACT_SILU: g / (1 + torch.exp(-g))}
    for kind, gate in gates.items():
        out = torch.zeros((rows, inner), dtype=torch.bfloat16, device=DEVICE)
        kn.gemm_tcgen05(x, w, out, rows, kn.TC_GATED + kind, flag, variant)
        want = gate * u
        bad = ((out.double() - want).abs() > 2.5e-2 * (1 + want.abs())).sum().item()
        assert bad <= rows * inner // 2000, (kind, bad)          # a gate on a rounding edge may flip
    plain = torch.zeros((rows, inner), dtype=torch.bfloat16, device=DEVICE)
    kn.gemm_tcgen05(x, w, plain, rows, kn.TC_SWIGLU, flag, variant)
    assert torch.equal(plain, out)                              # (the last kind above was SiLU)
    assert int(flag.item()) == 0
