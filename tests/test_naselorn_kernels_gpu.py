"""The kernels that the Naselorn design added, each against the same operation written in PyTorch (float64 on the
CPU): the gated norm over a wide row, the gated linear recurrent unit as a scan over portions and as one decoding
launch (which must agree with each other too), the sum of two mixers, activations of some columns, the gated product
with ReLU, biases into the paged cache, sinusoidal positions at the embedding, the retention's decoding step with an
activation on what it reads, and the router with a bias."""
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


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ----------------------------------------------------------------------------------------------- gated norm
@pytest.mark.parametrize("dtype,rel", [(torch.float32, 2e-6), (torch.bfloat16, 6e-3)])
@pytest.mark.parametrize("tokens,heads,vdim", [(5, 3, 40), (3, 1, 512), (9, 1, 2048), (4, 2, 515), (2, 1, 1028), (300, 1, 768)])
@pytest.mark.parametrize("gate_kind", ["sigmoid", "silu"])
def test_gated_norm_of_narrow_heads_and_wide_rows(tokens, heads, vdim, gate_kind, dtype, rel):
    k = kernels()
    rng = np.random.default_rng(tokens * 1000 + vdim)
    width = heads * vdim
    o = rng.normal(size=(tokens, width)) * 3.0
    rows = rng.normal(size=(tokens, width + 8))          # the gate is a slice of wider rows
    weight = rng.normal(1.0, 0.3, size=width)
    eps = 1e-5
    read = o.reshape(tokens, heads, vdim)
    normed = (read / np.sqrt((read ** 2).mean(-1, keepdims=True) + eps)).reshape(tokens, width) * weight
    z = rows[:, 8:]
    want = normed * (sigmoid(z) if gate_kind == "sigmoid" else z * sigmoid(z))
    out = torch.zeros((tokens, width), dtype=dtype, device=DEVICE)
    k.gated_head_norm(gpu(o), gpu(rows)[:, 8:], gpu(weight), True, out, tokens, heads, vdim, eps,
                      k.GATE_SIGMOID if gate_kind == "sigmoid" else k.GATE_SILU)
    close(out, want, rel, f"gated norm {tokens}x{heads}x{vdim} {gate_kind}")


# ----------------------------------------------------------------------------- gated linear recurrent unit
def plain_unit(proj, bias, taps, conv_bias, carried, state, gate_w, gate_bias, lam, c):
    """One sequence in float64. proj [tokens, 2 width] rows [y | x]; carried [n - 1, width] oldest first; returns
    (out [tokens, width], carried after, state after)."""
    tokens, width = proj.shape[0], proj.shape[1] // 2
    n = taps.shape[1]
    blocks, part = gate_w.shape[1], gate_w.shape[2]
    y = gelu_tanh(proj[:, :width] + bias[:width])
    x = proj[:, width:] + bias[width:]
    padded = np.concatenate([carried, x])
    u = sum(taps[:, j] * padded[j:j + tokens] for j in range(n)) + conv_bias
    out = np.zeros((tokens, width))
    soft = np.logaddexp(0.0, lam)
    for t in range(tokens):
        r, i = np.zeros(width), np.zeros(width)
        for b in range(blocks):
            cut = slice(b * part, (b + 1) * part)
            r[cut] = sigmoid(gate_w[0, b] @ u[t, cut] + gate_bias[:width][cut])
            i[cut] = sigmoid(gate_w[1, b] @ u[t, cut] + gate_bias[width:][cut])
        a = np.exp(-c * r * soft)
        state = a * state + np.sqrt(1.0 - a * a) * i * u[t]
        out[t] = state * y[t]
    return out, padded[tokens:], state


@pytest.mark.parametrize("dtype,rel", [(torch.float32, 2e-5), (torch.bfloat16, 6e-3)])
@pytest.mark.parametrize("width,blocks,n_taps,spans", [(16, 1, 1, [5]), (48, 3, 4, [1, 7, 2, 40]), (40, 4, 2, [3, 3]),
                                                       (132, 3, 7, [2, 90, 1]), (256, 2, 4, [700]), (35, 5, 3, [1, 1, 1, 1])])
def test_recurrent_unit_over_portions_and_token_by_token(width, blocks, n_taps, spans, dtype, rel):
    """Portions of unequal length in slots out of order, from states and carried inputs that are not zero: the scan's
    four launches against float64; then the same tokens one by one through the decoding launch, from the same start."""
    k = kernels()
    rng = np.random.default_rng(width + n_taps)
    part = width // blocks
    c = 8.0
    bias = rng.normal(0, 0.3, size=2 * width)
    taps = rng.normal(0, 0.5, size=(width, n_taps))
    conv_bias = rng.normal(0, 0.3, size=width)
    gate_w = rng.normal(0, 1.0 / math.sqrt(part), size=(2, blocks, part, part))
    gate_bias = rng.normal(0, 0.5, size=2 * width)
    lam = rng.uniform(-7.0, 1.0, size=width)
    slots = len(spans) + 2
    slot_of = rng.permutation(slots)[:len(spans)]
    elements = n_taps * width
    start = rng.normal(size=(slots, elements))
    tokens = sum(spans)
    proj = rng.normal(size=(tokens, 2 * width))
    begin = np.concatenate([[0], np.cumsum(spans)])
    want = np.zeros((tokens, width))
    after = start.copy()
    for s, length in enumerate(spans):
        slot = slot_of[s]
        carried = start[slot, :(n_taps - 1) * width].reshape(n_taps - 1, width)
        out, carried_after, state_after = plain_unit(proj[begin[s]:begin[s + 1]], bias, taps, conv_bias, carried,
                                                     start[slot, (n_taps - 1) * width:], gate_w, gate_bias, lam, c)
        want[begin[s]:begin[s + 1]] = out
        after[slot] = np.concatenate([carried_after.reshape(-1), state_after])
    args = dict(bias=gpu(bias), taps=gpu(taps), conv_bias=gpu(conv_bias), gate_w=gpu(gate_w), gate_bias=gpu(gate_bias), lam=gpu(lam))
    token_span = gpu(np.repeat(np.arange(len(spans)), spans), torch.int32)
    span_begin, span_slot = gpu(begin, torch.int32), gpu(slot_of, torch.int32)

    state = gpu(start)
    proj_d = gpu(proj)
    branch = torch.zeros((tokens, width), device=DEVICE)
    conved = torch.zeros((tokens, width), device=DEVICE)
    gates = torch.zeros((tokens, 2 * width), device=DEVICE)
    out = torch.zeros((tokens, width), dtype=dtype, device=DEVICE)
    k.lru_prepare(proj_d, args["bias"], args["taps"], args["conv_bias"], state, state.stride(0), token_span, span_begin,
                  span_slot, branch, conved, tokens, len(spans), width, n_taps)
    k.block_diagonal_product(conved, blocks, args["gate_w"].view(2 * blocks, part, part), gates, tokens)
    k.lru_scan(gates, conved, args["gate_bias"], args["lam"], c, branch, out, state[:, (n_taps - 1) * width:], state.stride(0),
               span_begin, span_slot, tokens, len(spans), width)
    close(out, want, rel, "scan over portions")
    close(state, after, 2e-5, "states and carried inputs after the portions")

    state = gpu(start)
    out = torch.zeros((tokens, width), dtype=dtype, device=DEVICE)
    longest = max(spans)
    for step in range(min(longest, 48)):
        live = [s for s, length in enumerate(spans) if step < length]
        rows = gpu(np.stack([proj[begin[s] + step] for s in live]))
        step_out = torch.zeros((len(live), width), dtype=dtype, device=DEVICE)
        k.lru_decode(rows, args["bias"], args["taps"], args["conv_bias"], state, state[:, (n_taps - 1) * width:], state.stride(0),
                     gpu(slot_of[live], torch.int32), args["gate_w"], args["gate_bias"], args["lam"], c, step_out, len(live),
                     width, n_taps, blocks)
        for row, s in enumerate(live):
            out[begin[s] + step] = step_out[row]
    decoded = np.concatenate([np.arange(begin[s], begin[s] + min(length, 48)) for s, length in enumerate(spans)])
    close(out[decoded], want[decoded], rel, "token by token")
    if longest <= 48:
        close(state, after, 2e-5, "states and carried inputs after decoding")


def test_block_diagonal_product_shares_its_input_between_both_gates():
    k = kernels()
    rng = np.random.default_rng(5)
    for rows, parts, n in ((7, 3, 10), (300, 2, 128), (65, 5, 33)):
        x = rng.normal(size=(rows, parts * n))
        w = rng.normal(size=(2 * parts, n, n))
        want = np.concatenate([x[:, (z % parts) * n:(z % parts + 1) * n] @ w[z].T for z in range(2 * parts)], axis=1)
        y = torch.zeros((rows, 2 * parts * n), device=DEVICE)
        k.block_diagonal_product(gpu(x), parts, gpu(w), y, rows)
        close(y, want, 3e-6, f"block-diagonal product {rows}x{parts}x{n}")


# ------------------------------------------------------------------------------------------- small launches
@pytest.mark.parametrize("dtype,rel", [(torch.float32, 1e-6), (torch.bfloat16, 5e-3)])
def test_scaled_sum_of_two_mixers_with_a_bias(dtype, rel):
    k = kernels()
    rng = np.random.default_rng(6)
    for rows, width in ((3, 36), (200, 128), (17, 1030)):
        a, b, bias = rng.normal(size=(rows, width)), rng.normal(size=(rows, width)), rng.normal(size=width)
        out = torch.zeros((rows, width), dtype=dtype, device=DEVICE)
        k.scaled_sum(gpu(a), gpu(b), gpu(bias), 1.25, -0.75, out, rows)
        close(out, 1.25 * (a + bias) - 0.75 * b, rel, "two terms and a bias")
        k.scaled_sum(gpu(a), None, gpu(bias), 1.0, 0.0, out, rows)
        close(out, a + bias, rel, "one term and a bias")
        k.scaled_sum(gpu(a), gpu(b), None, 0.5, 2.0, out, rows)
        close(out, 0.5 * a + 2.0 * b, rel, "two terms")


def test_activation_of_the_first_columns_only():
    k = kernels()
    rng = np.random.default_rng(7)
    for rows, width, columns in ((5, 50, 30), (300, 2048, 1536), (9, 131, 131)):
        x = rng.normal(size=(rows, width)) * 3.0
        want = x.copy()
        want[:, :columns] = x[:, :columns] * sigmoid(x[:, :columns])
        rows_d = gpu(x)
        k.activation_columns(rows_d, columns, rows, k.ACT_SILU)
        close(rows_d, want, 1e-6, f"SiLU of {columns} of {width} columns")


@pytest.mark.parametrize("dtype,rel", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)])
def test_gated_product_with_relu_and_with_silu(dtype, rel):
    k = kernels()
    rng = np.random.default_rng(8)
    for rows, inner in ((4, 44), (130, 256), (3, 2736)):
        both = rng.normal(size=(rows, 2 * inner))
        both_d = gpu(both, dtype)
        seen = both_d.float().cpu().numpy().astype(np.float64)
        gate, up = seen[:, :inner], seen[:, inner:]
        out = torch.zeros((rows, inner), dtype=dtype, device=DEVICE)
        k.glu(both_d, out, rows, inner, k.ACT_RELU)
        close(out, np.maximum(gate, 0.0) * up, rel, "ReLU gate")
        k.glu(both_d, out, rows, inner, k.ACT_SILU)
        close(out, gate * sigmoid(gate) * up, rel, "SiLU gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,dim,vdim,key_store,value_store", [(4, 2, 16, 32, 32, 32), (3, 1, 12, 7, 12, 7),
                                                                         (8, 1, 64, 128, 128, 128), (2, 2, 24, 8, 24, 8)])
def test_biases_are_added_on_the_way_into_the_paged_cache(heads, groups, dim, vdim, key_store, value_store, dtype):
    """Two requests' tokens at scattered positions; stored heads may be wider than projected ones (zeros behind)."""
    k = kernels()
    rng = np.random.default_rng(9)
    page_tokens, pages = 8, 12
    positions = np.array([0, 1, 2, 21, 22, 23, 24, 7])
    span = np.array([0, 0, 0, 1, 1, 1, 1, 0])
    table = np.full((2, 6), -1)
    table[0, :2] = [5, 3]
    table[1, :4] = [9, 0, 7, 2]
    tokens = len(positions)
    widths = (heads * dim, groups * dim, groups * vdim)
    proj = rng.normal(size=(tokens, sum(widths)))
    bias = rng.normal(size=sum(widths))
    q_out = torch.full((tokens, heads * key_store), 7.0, dtype=dtype, device=DEVICE)
    k_cache = torch.full((pages, groups, page_tokens, key_store), 7.0, dtype=dtype, device=DEVICE)
    v_cache = torch.full((pages, groups, page_tokens, value_store), 7.0, dtype=dtype, device=DEVICE)
    flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    k.bias_store_kv(gpu(proj), gpu(bias), q_out, gpu(positions, torch.int32), gpu(span, torch.int32), gpu(table, torch.int32),
                    k_cache, v_cache, tokens, heads, groups, dim, vdim, key_store, value_store, page_tokens, flag)
    assert int(flag.item()) == 0
    summed = proj + bias
    rel = 1e-6 if dtype == torch.float32 else 5e-3
    want_q = np.zeros((tokens, heads, key_store))
    want_q[:, :, :dim] = summed[:, :widths[0]].reshape(tokens, heads, dim)
    close(q_out, want_q.reshape(tokens, -1), rel, "queries")
    want_k = np.full((pages, groups, page_tokens, key_store), 7.0)
    want_v = np.full((pages, groups, page_tokens, value_store), 7.0)
    for t in range(tokens):
        page, at = table[span[t], positions[t] // page_tokens], positions[t] % page_tokens
        want_k[page, :, at] = 0.0
        want_k[page, :, at, :dim] = summed[t, widths[0]:widths[0] + widths[1]].reshape(groups, dim)
        want_v[page, :, at] = 0.0
        want_v[page, :, at, :vdim] = summed[t, widths[0] + widths[1]:].reshape(groups, vdim)
    close(k_cache, want_k, rel, "keys in their pages (other places untouched)")
    close(v_cache, want_v, rel, "values in their pages (other places untouched)")


def test_sinusoidal_positions_at_the_embedding():
    k = kernels()
    rng = np.random.default_rng(10)
    for width in (36, 64, 129):
        vocab = 50
        table = torch.as_tensor(rng.normal(size=(vocab, width))).to(torch.bfloat16)
        tokens = rng.integers(0, vocab, size=9)
        positions = np.array([0, 1, 2, 63, 64, 1000, 4095, 8191, 5])
        pairs = (width + 1) // 2
        frequencies = 10000.0 ** (-2.0 * np.arange(pairs) / width)
        want = table.double().numpy()[tokens] * 3.5
        for row, p in enumerate(positions):
            for i in range(pairs):
                angle = p * float(np.float32(frequencies[i]))
                want[row, 2 * i] += math.sin(angle)
                if 2 * i + 1 < width:
                    want[row, 2 * i + 1] += math.cos(angle)
        out = torch.zeros((9, width), device=DEVICE)
        k.embedding(table.to(DEVICE), gpu(tokens, torch.int32), out, 3.5, positions=gpu(positions, torch.int32),
                    frequencies=gpu(frequencies))
        assert np.abs(out.cpu().numpy() - want).max() <= 2e-3, f"width {width}"      # (a float32 angle of thousands)
        assert np.abs(out.cpu().numpy()[:5] - want[:5]).max() <= 2e-5


@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (3, 64, 128), (1, 136, 8), (4, 8, 5)])
def test_retention_step_with_silu_on_what_it_reads(heads, dim, vdim):
    """S <- d S + silu(k) silu(v)^T, read-out S^T silu(q), the read-outs left as they are; requests in slots out of
    order, states that are not zero."""
    k = kernels()
    rng = np.random.default_rng(11)
    requests, slots = 5, 7
    width, v_width = heads * dim, heads * vdim
    proj = rng.normal(size=(requests, 2 * width + 2 * v_width))
    decay = rng.uniform(0.5, 1.0, size=heads)
    decay[-1] = 1.0
    start = rng.normal(size=(slots, heads, dim, vdim))
    slot_of = rng.permutation(slots)[:requests]
    silu = lambda z: z * sigmoid(z)
    q = silu(proj[:, :width]).reshape(requests, heads, dim)
    key = silu(proj[:, width:2 * width]).reshape(requests, heads, dim)
    v = silu(proj[:, 2 * width:2 * width + v_width]).reshape(requests, heads, vdim)
    after = start.copy()
    want = np.zeros((requests, heads, vdim))
    for r in range(requests):
        for h in range(heads):
            s = decay[h] * start[slot_of[r], h] + np.outer(key[r, h], v[r, h])
            after[slot_of[r], h] = s
            want[r, h] = s.T @ q[r, h]
    state = gpu(start.reshape(slots, -1))
    read = torch.zeros((requests, v_width), device=DEVICE)
    k.retention_decode_raw(gpu(proj), (0, width, 2 * width), gpu(decay), state, state.stride(0), gpu(slot_of, torch.int32),
                           requests, heads, dim, vdim, 1.0, k.ACT_SILU, read)
    close(read, want.reshape(requests, -1), 3e-6, "read-outs")
    close(state, after.reshape(slots, -1), 3e-6, "states")


def test_router_bias_enters_the_choice_and_the_weights():
    k = kernels()
    rng = np.random.default_rng(12)
    for tokens, experts, top in ((6, 8, 3), (40, 40, 5), (3, 5, 5), (9, 6, 1)):
        logits = rng.normal(size=(tokens, experts)) * 2.0
        bias = rng.normal(size=experts) * 2.0
        total = logits + bias
        order = np.argsort(-total, axis=-1, kind="stable")[:, :top]
        picked = np.take_along_axis(total, order, axis=-1)
        weights = np.exp(picked - picked.max(-1, keepdims=True))
        weights /= weights.sum(-1, keepdims=True)
        chosen_d = torch.zeros((tokens, top), dtype=torch.int32, device=DEVICE)
        weights_d = torch.zeros((tokens, top), device=DEVICE)
        k.moe_route(gpu(logits), experts, None, None, chosen_d, weights_d, None, tokens, top, bias=gpu(bias))
        got = chosen_d.cpu().numpy()
        got_w = weights_d.cpu().numpy().astype(np.float64)
        for t in range(tokens):
            assert set(got[t]) == set(order[t]), f"token {t}: chose {got[t]}, wanted {order[t]}"
            by_expert = dict(zip(order[t], weights[t]))
            assert all(abs(got_w[t, j] - by_expert[got[t, j]]) <= 2e-6 for j in range(top))


def test_weight_streaming_gated_product_with_another_gate_function():
    """Few rows: [gate | up] product and the gate's function in one launch; ReLU and the tanh GELU beside SiLU."""
    k = kernels()
    rng = np.random.default_rng(13)
    for rows, width, inner in ((1, 64, 48), (8, 256, 352), (16, 128, 136)):
        x = gpu(rng.normal(size=(rows, width)), torch.bfloat16)
        w = gpu(rng.normal(size=(2 * inner, width)) / math.sqrt(width), torch.bfloat16)
        assert k.gemv_supported(rows, x, w)
        sums = x.double().cpu().numpy() @ w.double().cpu().numpy().T
        sums = torch.as_tensor(sums).to(torch.bfloat16).double().numpy()          # both halves are rounded as if stored
        gate, up = sums[:, :inner], sums[:, inner:]
        for kind, function in ((k.ACT_SILU, lambda z: z * sigmoid(z)), (k.ACT_RELU, lambda z: np.maximum(z, 0.0)),
                               (k.ACT_GELU_TANH, gelu_tanh)):
            out = torch.zeros((rows, inner), dtype=torch.bfloat16, device=DEVICE)
            k.gemv_bf16(x, w, out, rows, k.GEMV_SWIGLU, taps=0 if kind == k.ACT_SILU else 1 + kind)
            close(out, function(gate) * up, 1.2e-2, f"gate function {kind} at {rows}x{width}x{inner}")
