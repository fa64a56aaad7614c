"""GPU tests of the Talapel architecture: every mechanism's kernel against oracle/talapel.py (plain numpy, float64), then the
engine — whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with reused pages and state
slots, long decoding, greedy generation through LLMEngine.generate and a replay through bin/trace_run — on small random
models.  f32 engines must agree with the oracle to rounding; bf16 engines within the error of bf16 operands."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import talapel as T

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
F32 = torch.float32


def within(e, dtype):
    """f32: every position to rounding.  bf16: operand rounding through several looped layers of a 24-wide model scatters
    (a few positions reach 0.1 of a row's spread while the typical one stays near 0.02); a wrong key, state or page moves
    whole rows by O(1)."""
    e = np.asarray(e)
    if not np.isfinite(e).all():
        return False
    return e.max() < TOL[dtype] if dtype == "float32" else (e.max() < 0.2 and e.mean() < 0.05)


def dev_t(a, dev, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).to(dtype)


def dev_i(a, dev, dtype=torch.int32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(dtype)


def rel_err(got, ref):
    """Per row: rms of the centred difference over the rms of the centred reference."""
    d = np.asarray(got, np.float64) - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((r ** 2).mean(-1))


# ------------------------------------------------------------------------------------------------ mechanisms alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hid", [50, 256, 1])
def test_residual_layernorm(cuda, dtype, hid):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(hid)
    n, eps = 13, 1e-3
    h = rng.standard_normal((n, hid)) * 3 + 1.5
    a0, a1 = rng.standard_normal((n, hid)), rng.standard_normal((n, hid))
    a2 = T.bf16_round(rng.standard_normal((n, hid)))
    bias, w = rng.standard_normal(hid), rng.standard_normal(hid)
    hd = dev_t(h, cuda)
    out = ops.residual_layernorm(hd, [(dev_t(a0, cuda), 1.2), (dev_t(a1, cuda), -0.7), (dev_t(a2, cuda, dtype), 1.0)], dev_t(bias, cuda), 1.2,
                                 dev_t(w, cuda), eps, dtype)
    f = lambda x: x.astype(np.float32).astype(np.float64)
    h_ref = f(h) + 1.2 * f(a0) - 0.7 * f(a1) + a2 + 1.2 * f(bias)
    np.testing.assert_allclose(hd.cpu().numpy(), h_ref, rtol=3e-6, atol=3e-6)
    ref = np.stack([T.layer_norm(r, f(w), eps) for r in h_ref])
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=1e-2 if dtype == torch.bfloat16 else 2e-5, atol=2e-5 if dtype == F32 else 1e-2)
    # the sum alone (no norm) and the norm alone (no addends) compose to the same
    h2 = dev_t(h, cuda)
    assert ops.residual_layernorm(h2, [(dev_t(a0, cuda), 1.2), (dev_t(a1, cuda), -0.7), (dev_t(a2, cuda, dtype), 1.0)], dev_t(bias, cuda), 1.2) is None
    assert torch.equal(h2, hd)
    assert torch.equal(ops.residual_layernorm(h2, weight=dev_t(w, cuda), eps=eps, dtype=dtype), out) and torch.equal(h2, hd)


def test_concat_embedding_activation_table_route(cuda):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(2)
    a, b = rng.standard_normal((5, 7)), rng.standard_normal((5, 3))
    for dt in (torch.float32, torch.bfloat16):
        c = ops.concat_cast(dev_t(a, cuda), dev_t(b, cuda), dt).float().cpu().numpy()
        np.testing.assert_allclose(c, np.concatenate([a, b], 1), rtol=1e-2 if dt == torch.bfloat16 else 1e-6)
    table = T.bf16_round(rng.standard_normal((11, 6)))
    ids = np.array([3, 0, 10, 3])
    for dt in (torch.float32, torch.bfloat16):
        h, h2 = ops.embedding_gather_scaled(dev_t(table, cuda, dt), dev_i(ids, cuda, torch.int64), 2.5, copy=True)
        np.testing.assert_allclose(h.cpu().numpy(), table[ids] * 2.5, rtol=1e-6)
        assert torch.equal(h, h2)
    x = rng.standard_normal((9, 10))
    got = ops.ff_activation(dev_t(x, cuda), 0).cpu().numpy()
    np.testing.assert_allclose(got, T.silu(x[:, :5]) * x[:, 5:], rtol=1e-5, atol=1e-6)
    got = ops.ff_activation(dev_t(x, cuda), 1).cpu().numpy()
    np.testing.assert_allclose(got, np.maximum(x, 0) ** 2, rtol=1e-5, atol=1e-6)
    tab = np.stack([rng.permutation(7)[:3] for _ in range(11)]).astype(np.int32)
    idx, w = ops.moe_table_route(dev_i(tab, cuda), dev_i(ids, cuda, torch.int64))
    assert np.array_equal(idx.cpu().numpy(), tab[ids]) and np.allclose(w.cpu().numpy(), 1 / 3)


def _paged(rng, ctxs, bs, spare=3):
    """Random page assignment: tables [seqs, cap], and for every (sequence, position) its cache slot."""
    need = [(c + bs - 1) // bs for c in ctxs]
    perm = rng.permutation(sum(need) + spare)
    cap = max(need) + 1
    tables = -np.ones((len(ctxs), cap), np.int32)
    k = 0
    for s, nb in enumerate(need):
        tables[s, :nb] = perm[k:k + nb]; k += nb
    slot = lambda s, p: int(tables[s, p // bs]) * bs + p % bs
    return tables, slot, (sum(need) + spare) * bs


def _attention_ref(q, keys, vals, m, pos):
    """q [H, D] already biased; keys / vals: lists of [G, D] / [G, V] up to and including pos."""
    H, G = m["heads"], m["kv_heads"]
    out = np.zeros((H, m["vdim"]))
    qt = q * T.query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"])
    for h in range(H):
        g = h // (H // G)
        s = np.array([qt[h] @ k[g] for k in keys]) * m["scale"]
        if m["softcap"] > 0:
            s = m["softcap"] * np.tanh(s / m["softcap"])
        e = np.exp(s - s.max()); e /= e.sum()
        out[h] = sum(p * v[g] for p, v in zip(e, vals))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V", [(4, 2, 6, 10), (3, 3, 16, 16), (5, 1, 40, 33), (8, 2, 40, 88), (6, 2, 64, 32), (2, 1, 128, 128), (1, 1, 12, 300)])
def test_capped_attention_paged(cuda, dtype, H, G, D, V):
    """Prompt portions and single tokens of three sequences in one launch, pages in random order, query positions around the
    temperature steps and the page borders; biases, the gate and the cache store included.  bf16 with head sizes that are
    multiples of 8 runs on the tensor-core kernel (groups of 1, 3, 4 and 2 heads per key head), the rest one warp per row."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(H * 100 + D)
    bs, every = 8, 5
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.4, "softcap": 3.0, "q_temp": {"coef": 0.6, "every": every}}
    ctx = [41, 9, 24]                      # tokens each sequence ends with
    new = [17, 1, 24]                      # of which the step brings the last `new`
    tables, slot, nslots = _paged(rng, ctx, bs)
    rd = lambda *s: T.bf16_round(rng.standard_normal(s)) if dtype == torch.bfloat16 else rng.standard_normal(s)
    K = [rd(c, G, D) for c in ctx]; Vv = [rd(c, G, V) for c in ctx]
    kc = torch.zeros((nslots, G * D + 8), dtype=dtype, device=cuda); vc = torch.zeros((nslots, G * V), dtype=dtype, device=cuda)
    qb, kb, vb = rng.standard_normal(H * D), rng.standard_normal(G * D), rng.standard_normal(G * V)
    proj, slots, tok_seq, pos = [], [], [], []
    for s, (c, n) in enumerate(zip(ctx, new)):
        for p in range(c - n):             # earlier tokens are in the cache already
            kc[slot(s, p), :G * D] = dev_t(K[s][p].reshape(-1), cuda, dtype); vc[slot(s, p)] = dev_t(Vv[s][p].reshape(-1), cuda, dtype)
        for p in range(c - n, c):
            q = rng.standard_normal(H * D)
            proj.append(np.concatenate([q, K[s][p].reshape(-1) - kb, Vv[s][p].reshape(-1) - vb, rng.standard_normal(H * V), [7.0]]))
            slots.append(slot(s, p)); tok_seq.append(s); pos.append(p)
    proj = np.array(proj)
    pd = dev_t(proj, cuda)
    qd = ops.attn_bias_store(pd, H * D, G * D, G * V, dev_t(qb, cuda), dev_t(kb, cuda), dev_t(vb, cuda), kc, vc, dev_i(slots, cuda), dtype)
    gate = pd[:, H * D + G * D + G * V:]
    out = ops.capped_attention(qd, gate, kc, vc, dev_i(tok_seq, cuda), dev_i(pos, cuda, torch.int64), dev_i(tables, cuda), bs, H, G, D, V,
                               m["scale"], m["softcap"], 0.6, every, cu_tokens=dev_i(np.concatenate([[0], np.cumsum(new)]), cuda)).float().cpu().numpy()
    if dtype == torch.bfloat16:   # the kernel without the token ranges (one warp per row) agrees with the tensor-core one
        plain = ops.capped_attention(qd, gate, kc, vc, dev_i(tok_seq, cuda), dev_i(pos, cuda, torch.int64), dev_i(tables, cuda), bs, H, G, D, V,
                                     m["scale"], m["softcap"], 0.6, every).float().cpu().numpy()
        np.testing.assert_allclose(out, plain, rtol=2e-2, atol=2e-2)
    qs = qd.float().cpu().numpy().astype(np.float64)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    for i, (s, p) in enumerate(zip(tok_seq, pos)):
        kk = [kc[slot(s, j), :G * D].float().cpu().numpy().astype(np.float64).reshape(G, D) for j in range(p + 1)]
        vv = [vc[slot(s, j)].float().cpu().numpy().astype(np.float64).reshape(G, V) for j in range(p + 1)]
        if dtype == torch.float32:         # the store added the biases: rows equal the intended keys
            np.testing.assert_allclose(kk[p], K[s][p], rtol=1e-5, atol=1e-5)
        ref = _attention_ref(qs[i].reshape(H, D), kk, vv, m, p).reshape(-1)
        ref = ref / (1 + np.exp(-proj[i, H * D + G * D + G * V:-1].astype(np.float32).astype(np.float64)))
        np.testing.assert_allclose(out[i], ref, rtol=tol, atol=tol, err_msg=f"token {i} seq {s} pos {p}")
    assert torch.all(kc[:, G * D:] == 0)   # the row padding stays untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("where", ["first", "far", "page_end", "page_start", "last", "next"])
def test_capped_attention_one_key_stands_out(cuda, where, dtype):
    """One key among 300 is aligned with the query so that its (capped) score dominates: the output must be that key's value —
    unless it lies in the future (`next`)."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(7)
    H, G, D, V, bs, ctx = 2, 1, 16, 16, 16, 300
    qpos = 250
    at = {"first": 0, "far": 37, "page_end": 16 * 9 + 15, "page_start": 16 * 10, "last": qpos, "next": qpos + 1}[where]
    tables, slot, nslots = _paged(rng, [ctx], bs)
    K = T.bf16_round(rng.standard_normal((ctx, D)) * 0.1); Vv = T.bf16_round(rng.standard_normal((ctx, V)))
    q = T.bf16_round(rng.standard_normal((H, D)))
    K[at] = q[1] * 4.0                                   # head 1's query points at key `at`
    kc = torch.zeros((nslots, D), dtype=dtype, device=cuda); vc = torch.zeros((nslots, V), dtype=dtype, device=cuda)
    for p in range(ctx):
        kc[slot(0, p)] = dev_t(K[p], cuda, dtype); vc[slot(0, p)] = dev_t(Vv[p], cuda, dtype)
    out = ops.capped_attention(dev_t(q.reshape(1, -1), cuda, dtype), None, kc, vc, dev_i([0], cuda), dev_i([qpos], cuda, torch.int64),
                               dev_i(tables, cuda), bs, H, G, D, V, 1.0, 20.0, 0.0, 1,
                               cu_tokens=dev_i([0, 1], cuda)).float().cpu().numpy().reshape(H, V)   # bf16: tensor cores
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 1.0, "softcap": 20.0, "q_temp": {"coef": 0.0, "every": 1}}
    ref = _attention_ref(q, [k[None] for k in K[:qpos + 1]], [v[None] for v in Vv[:qpos + 1]], m, qpos)
    np.testing.assert_allclose(out, ref, rtol=2e-2, atol=2e-2)
    if where == "next":
        assert np.abs(out[1] - Vv[at]).max() > 0.3        # the future key must not show
    else:
        np.testing.assert_allclose(out[1], Vv[at], atol=2e-2)


def _steps_meta(lens, starts, slots, dev):
    """Step metadata of a batch of sequences: token i of sequence s has position starts[s] + i."""
    tok_seq = np.concatenate([[s] * n for s, n in enumerate(lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(st, st + n) for st, n in zip(starts, lens)]).astype(np.int64)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    return dev_i(tok_seq, dev), dev_i(slots, dev), dev_i(cu, dev), dev_i(pos, dev, torch.int64)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_conv_carries_its_last_inputs(cuda, taps):
    """Two sequences cut into portions of 1..9 tokens (shorter than the window too) in slots that hold leftovers: equal to the
    convolution of the whole sequence with zeros before its start."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(taps)
    ch, lens = 11, [23, 14]
    x = [rng.standard_normal((n, ch + 2)) for n in lens]       # two extra columns: the kernel reads a strided view
    w, b = rng.standard_normal((ch, taps)), rng.standard_normal(ch)
    state = torch.full((4, max(taps - 1, 1), ch), 9.0, device=cuda)          # garbage from an earlier user of the slots
    ref = []
    for xs in x:
        pad = np.vstack([np.zeros((taps - 1, ch)), xs[:, :ch]])
        ref.append(T.silu(np.stack([(pad[t:t + taps] * w.T).sum(0) + b for t in range(len(xs))])))
    at, got = [0, 0], [[], []]
    cuts = [[1, 2, 9, 1, 1, 3, 6], [5, 1, 1, 2, 5]]
    for k in range(7):
        seqs = [s for s in (0, 1) if k < len(cuts[s])]
        ls = [cuts[s][k] for s in seqs]
        xin = dev_t(np.vstack([x[s][at[s]:at[s] + n] for s, n in zip(seqs, ls)]), cuda)
        meta = _steps_meta(ls, [at[s] for s in seqs], [3 - 2 * s for s in seqs], cuda)
        out = ops.causal_conv(xin[:, :ch], dev_t(w, cuda), dev_t(b, cuda), state, *meta).cpu().numpy()
        o = 0
        for s, n in zip(seqs, ls):
            got[s].append(out[o:o + n]); o += n; at[s] += n
    for s in (0, 1):
        np.testing.assert_allclose(np.vstack(got[s]), ref[s], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("heads,groups,dk,dv", [(4, 2, 5, 4), (3, 3, 16, 7), (2, 1, 48, 40), (1, 1, 130, 33), (2, 2, 64, 64), (1, 1, 300, 6)])
def test_linear_recurrence_portions_and_slots(cuda, heads, groups, dk, dv):
    """S <- a S + b k v^T, y = S^T q + d v with per-token decay and step: three sequences in portions of changing size through
    reused slots against the token-by-token recurrence in float64."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(dk)
    lens = [37, 5, 18]
    mk = lambda n, c: rng.standard_normal((n, c))
    q = [mk(n, groups * dk) for n in lens]; k = [mk(n, groups * dk) * 0.3 for n in lens]; v = [mk(n, heads * dv) for n in lens]
    a = [rng.uniform(0.7, 1.0, (n, heads)) for n in lens]; b = [rng.uniform(0.1, 1.0, (n, heads)) for n in lens]
    d = rng.standard_normal(heads)
    ref = []
    for s, n in enumerate(lens):
        S = np.zeros((heads, dk, dv)); ys = []
        for t in range(n):
            y = np.zeros((heads, dv))
            for h in range(heads):
                g = h // (heads // groups)
                vv = v[s][t, h * dv:(h + 1) * dv]
                S[h] = a[s][t, h] * S[h] + b[s][t, h] * np.outer(k[s][t, g * dk:(g + 1) * dk], vv)
                y[h] = S[h].T @ q[s][t, g * dk:(g + 1) * dk] + d[h] * vv
            ys.append(y.reshape(-1))
        ref.append(np.array(ys))
    state = torch.full((3, heads, dk, dv), 5.0, device=cuda)   # leftovers of an earlier sequence: a portion at position 0 ignores them
    cuts = [[2, 16, 1, 17, 1], [5], [1, 1, 14, 2]]
    slots = [2, 0, 0]                                          # sequence 2 takes slot 0 after sequence 1 is done
    at, got = [0] * 3, [[] for _ in lens]
    order = [[0, 1], [0], [0, 2], [0, 2], [0, 2], [2]]
    kk = [0] * 3
    for step in order:
        ls = [cuts[s][kk[s]] for s in step]
        cat = lambda arrs: dev_t(np.vstack([arrs[s][at[s]:at[s] + n] for s, n in zip(step, ls)]), cuda)
        meta = _steps_meta(ls, [at[s] for s in step], [slots[s] for s in step], cuda)
        y = ops.linear_recurrence(cat(q), cat(k), cat(v), cat(a), state, meta[1], meta[2], meta[3], heads, groups, dk, dv, step=cat(b),
                                  skip=dev_t(d, cuda)).cpu().numpy()
        o = 0
        for s, n in zip(step, ls):
            got[s].append(y[o:o + n]); o += n; at[s] += n; kk[s] += 1
    for s in range(3):
        assert at[s] == lens[s]
        np.testing.assert_allclose(np.vstack(got[s]), ref[s], rtol=2e-4, atol=2e-4)


def test_linear_recurrence_constant_decay_far_token(cuda):
    """Retention form (decay per head, no step, no skip): a token 400 steps back whose key equals the query still shows in the
    output of a slowly decaying head, scaled by decay^400, and is gone from a fast one."""
    from nano_vllm_rs_b200 import ops
    heads, dk, dv, n = 2, 8, 6, 420
    rng = np.random.default_rng(3)
    decay = np.array([0.999, 0.9])
    q = np.zeros((n, heads * dk)); k = rng.standard_normal((n, heads * dk)) * 1e-3; v = rng.standard_normal((n, heads * dv))
    probe = rng.standard_normal(dk)
    probe /= np.linalg.norm(probe)
    k[15, :dk] = k[15, dk:] = probe
    q[415, :dk] = q[415, dk:] = probe
    state = torch.zeros((1, heads, dk, dv), device=cuda)
    meta = _steps_meta([n], [0], [0], cuda)
    y = ops.linear_recurrence(dev_t(q, cuda), dev_t(k, cuda), dev_t(v, cuda), dev_t(decay, cuda), state, meta[1], meta[2], meta[3], heads,
                              heads, dk, dv).cpu().numpy()
    np.testing.assert_allclose(y[415, :dv], decay[0] ** 400 * v[15, :dv], atol=0.05)
    assert np.abs(y[415, dv:]).max() < 0.05 and np.abs(y[414]).max() == 0.0


def test_ssd_prepare_and_rotate_half(cuda):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(5)
    raw = rng.standard_normal((9, 6)) * 8                      # wide range: softplus must neither overflow nor vanish early
    bias, alog = rng.standard_normal(3), rng.uniform(-2, 1, 3)
    step, dec = ops.ssd_prepare(dev_t(raw, cuda)[:, 2:5], dev_t(bias, cuda), dev_t(alog, cuda))
    f = lambda x: np.asarray(x, np.float32).astype(np.float64)
    dt = T.softplus(f(raw)[:, 2:5] + f(bias))
    np.testing.assert_allclose(step.cpu().numpy(), dt, rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(dec.cpu().numpy(), np.exp(-np.exp(f(alog)) * dt), rtol=1e-5, atol=1e-7)
    Hh, dim, dims, base = 3, 10, 6, 777.0                      # dims < dim: the tail passes (scaled) unchanged
    pos = np.array([0, 1, 2, 63, 64, 65, 500, 1999, 7])
    x = rng.standard_normal((len(pos), Hh * dim + 4))
    tab = ops.rope_table_interleaved(2000, dims, base, cuda)
    xd = dev_t(x, cuda)
    ops.rotate_half(xd[:, 4:], dev_i(pos, cuda, torch.int64), tab, Hh, dim, dims, 0.5)
    got = xd.cpu().numpy()
    np.testing.assert_array_equal(got[:, :4], x.astype(np.float32)[:, :4])
    for t, p in enumerate(pos):
        ref = T.rotate_half(f(x[t, 4:]).reshape(Hh, dim), p, dims, base) * 0.5
        np.testing.assert_allclose(got[t, 4:].reshape(Hh, dim), ref, rtol=1e-5, atol=2e-5)
    y = dev_t(x, cuda)
    ops.rotate_half(y[:, 4:], dev_i(pos, cuda, torch.int64), None, Hh, dim, 0, 1.0)   # no rotated dimensions, no scale: untouched
    assert torch.equal(y, dev_t(x, cuda))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols,parts", [(16, 2), (30, 3), (7, 1), (512, 2)])
def test_gated_group_norm_both_orders(cuda, dtype, cols, parts):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(cols)
    n, eps = 6, 1e-3
    off = 4 if cols % 4 == 0 else 3      # 16-byte aligned views take the one-pass vector kernel
    y, z, w = rng.standard_normal((n, cols)), rng.standard_normal((n, cols + off)), rng.standard_normal(cols)
    f = lambda x: np.asarray(x, np.float32).astype(np.float64)
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-5
    first = ops.gated_group_norm(dev_t(y, cuda), dev_t(z, cuda)[:, off:], dev_t(w, cuda), parts, eps, True, dtype).float().cpu().numpy()
    t = f(y) * T.silu(f(z)[:, off:])
    ref = np.stack([np.concatenate([T.rms(p, eps) for p in np.split(r, parts)]) for r in t]) * f(w)
    np.testing.assert_allclose(first, ref, rtol=tol, atol=tol)
    after = ops.gated_group_norm(dev_t(y, cuda), dev_t(z, cuda)[:, off:], None, parts, eps, False, dtype).float().cpu().numpy()
    ref = np.stack([np.concatenate([T.rms(p, eps) for p in np.split(r, parts)]) for r in f(y)]) * T.silu(f(z)[:, off:])
    np.testing.assert_allclose(after, ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_table_experts_grouped(cuda, dtype):
    """Table routing -> sort by expert -> up projection with the squared-ReLU epilogue -> down -> combine, against the oracle."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(8)
    n, W, ff, E, top, vocab = 45, 20, 12, 5, 3, 30
    f = {"router": {"experts": E, "top": top}}
    w = {"table": np.stack([rng.permutation(E)[:top] for _ in range(vocab)]).astype(np.int32)}
    for e in range(E):
        w["e%d.up" % e] = T.bf16_round(rng.standard_normal((ff, W)) / 4); w["e%d.down" % e] = T.bf16_round(rng.standard_normal((W, ff)) / 3)
    ids = rng.integers(0, vocab, n)
    x = T.bf16_round(rng.standard_normal((n, W)))
    idx, wt = ops.moe_table_route(dev_i(w["table"], cuda), dev_i(ids, cuda, torch.int64))
    row_token, tile_expert, slot_row = ops.moe_sort(idx, E, 32)
    up = dev_t(np.concatenate([w["e%d.up" % e] for e in range(E)]), cuda, dtype)
    down = dev_t(np.concatenate([w["e%d.down" % e] for e in range(E)]), cuda, dtype)
    xd = dev_t(x, cuda, dtype)
    act = ops.linear_grouped(xd, up, row_token, tile_expert, row_token.shape[0], ff, W, ff * W, glu=2)
    eo = ops.linear_grouped(act, down, None, tile_expert, row_token.shape[0], W, ff, W * ff)
    out = ops.moe_combine(eo, xd, None, idx, wt, slot_row, E).float().cpu().numpy()
    ref = np.stack([T.table_experts(x[t], w, "", f, ids[t]) for t in range(n)])
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-5
    np.testing.assert_allclose(out, ref, rtol=tol, atol=tol)


# ------------------------------------------------------------------------------------------------ the engine

ATT = dict(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.35, softcap=4.0, coef=0.5, every=7)
SSD = dict(s_heads=4, groups=2, state=5, s_vdim=4, taps=3, norm_groups=2)


def variant(name):
    P, R = T.parallel_mixer, T.retention_mixer
    if name == "all_kinds":      # every layer kind, every feed-forward kind on both mixers, a loop over the middle
        return T.make_config([("parallel", P(**ATT, **SSD), T.dense_mlp(20)), ("retention", R(), T.expert_mlp()),
                              ("parallel", P(**ATT, **SSD, left_scale=0.7, right_scale=1.6), T.expert_mlp(4, 3, 9)),
                              ("retention", R(heads=2, dim=10, vdim=7, rot_dims=10, rot_base=31.0), None)], loop=(1, 3, 2))
    if name == "ones":           # sizes that are 1 or equal to one another, no loop, no cap, a window of one tap
        return T.make_config([("retention", R(heads=1, dim=6, vdim=6, rot_dims=0, decay=[0.9]), T.dense_mlp(8)),
                              ("parallel", P(heads=3, kv_heads=3, dim=8, vdim=8, softcap=0.0, coef=0.0, every=1, s_heads=1, groups=1, state=1,
                                             s_vdim=8, taps=1, norm_groups=1), T.expert_mlp(3, 1, 5)),
                              ("parallel", P(heads=1, kv_heads=1, dim=5, vdim=3, every=1, s_heads=2, groups=2, state=7, s_vdim=3, taps=2,
                                             norm_groups=3), None)], width=16, vocab=33, embed_scale=1.0)
    if name == "tensor_core":    # sizes the tensor-core GEMMs accept (bf16): width and inner sizes multiples of 64, experts of 64
        return T.make_config([("parallel", P(heads=2, kv_heads=1, dim=32, vdim=32, scale=0.2, softcap=10.0, coef=0.3, every=16, s_heads=4,
                                             groups=1, state=16, s_vdim=16, taps=4, norm_groups=2), T.expert_mlp(4, 2, 64)),
                              ("retention", R(heads=2, dim=32, vdim=32, rot_dims=16, rot_base=1e4), T.dense_mlp(128))],   # 128: SiLU gate in the GEMM epilogue
                             width=64, vocab=96, loop=(0, 2, 3))
    raise KeyError(name)


VARIANTS = ["all_kinds", "ones", "tensor_core"]


def make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=24, max_seqs=4, eager=1):
    from nano_vllm_rs_b200.engine import LLMEngine
    from nano_vllm_rs_b200.loader import write_safetensors
    d = tmp_path / ("m_" + dtype)
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: T.to_bf16_bits(v) for k, v in w.items()})
    return LLMEngine.from_pretrained(str(d), dtype=dtype, kvcache_block_size=bs, num_kvcache_blocks=blocks, max_num_seqs=max_seqs,
                                     max_num_batched_tokens=blocks * bs, max_model_len=blocks * bs, enforce_eager=eager), str(d)


def replay(eng, requests, schedule):
    """schedule: list of steps, each a list of (request index, token count).  Returns every position's logits per request."""
    from nano_vllm_rs_b200.engine import SamplingParams
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    sid, at, out = {}, {}, {i: [] for i in range(len(requests))}
    for step in schedule:
        ids, counts = [], []
        for i, c in step:
            toks = requests[i][at.get(i, 0):at.get(i, 0) + c]
            if i in sid:
                eng.scheduler.extend_sequence(sid[i], toks)
            else:
                sid[i] = eng.scheduler.add_sequence(toks, sp)
            ids.append(sid[i]); counts.append(c)
        lg = eng.step_chunks(ids, counts, list(range(sum(counts))))
        k = 0
        for i, c in step:
            out[i].append(lg[k:k + c]); k += c
            at[i] = at.get(i, 0) + c
            if at[i] == len(requests[i]):
                eng.scheduler.finish_sequence(sid[i]); eng.scheduler.release_sequence(sid[i])
                del sid[i]
    return {i: np.concatenate(v) for i, v in out.items()}


def cut(n, sizes):
    out, k = [], 0
    while n > 0:
        c = min(n, sizes[k % len(sizes)]); out.append(c); n -= c; k += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", VARIANTS)
def test_engine_schedules_match_the_oracle(cuda, tmp_path, name, dtype):
    rng = np.random.default_rng(100 + VARIANTS.index(name))
    cfg = variant(name)
    w = T.random_weights(cfg, rng)
    lens = [1, 2, 37, 70, 33]
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in lens]
    ref = [T.logits_of(cfg, w, r) for r in reqs]
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=12)    # 192 slots: the requests only fit one after another
    tol = TOL[dtype]

    def check(got, what):
        for i, r in enumerate(ref):
            e = rel_err(got[i], r)
            assert within(e, dtype), f"{name} {dtype} {what}: request {i} position {int(e.argmax())} error {e.max():.3g}"

    whole = replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    check(whole, "whole prompts")
    # most of the prompt at once, the last tokens one by one (decoding through cache and state across page borders)
    dec = replay(eng, reqs, [s for i, r in enumerate(reqs) for s in ([[(i, max(1, len(r) - 20))]] + [[(i, 1)]] * (len(r) - max(1, len(r) - 20)))])
    check(dec, "prefill + single tokens")
    one = replay(eng, reqs[:3], [[(i, 1)] for i, r in enumerate(reqs[:3]) for _ in r])
    for i in range(3):
        assert within(rel_err(one[i], ref[i]), dtype)
    # portions of changing size down to two tokens (shorter than the convolution window, across page and temperature steps)
    por = replay(eng, reqs, [[(i, c)] for i, r in enumerate(reqs) for c in cut(len(r), [2, 5, 16, 3, 17, 2, 31])])
    check(por, "portions")
    for i in range(len(reqs)):  # a position must not depend on how the prompt was cut, beyond rounding
        assert rel_err(por[i], whole[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else 0.2)
        assert rel_err(dec[i], whole[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else 0.2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_mixed_batches_reuse_pages_and_state_slots(cuda, tmp_path, dtype):
    """Up to four live requests per step, portions of some beside single tokens of others, in a pool that only holds them
    because finished requests give their pages and state slots back; every request equals its run alone and the oracle."""
    rng = np.random.default_rng(11)
    cfg = variant("all_kinds")
    w = T.random_weights(cfg, rng)
    lens = [50, 23, 64, 9, 41, 30, 17]
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in lens]
    ref = [T.logits_of(cfg, w, r) for r in reqs]
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=11, max_seqs=4)   # 176 slots < 234 tokens in total
    need = [(n + 15) // 16 for n in lens]
    at, live, nxt, sched, k = [0] * len(lens), [], 0, [], 0
    while nxt < len(reqs) or live:
        while nxt < len(reqs) and len(live) < 4 and sum(need[i] for i in live) + need[nxt] <= 11:
            live.append(nxt); nxt += 1
        step = []
        for i in live:
            k += 1
            if k % 5 == 0 and len(live) > 1:
                continue                                  # a live request may sit a step out
            c = 1 if (at[i] > lens[i] // 2 or k % 3 == 0) else [2, 7, 16, 5][k % 4]
            c = min(c, lens[i] - at[i])
            step.append((i, c)); at[i] += c
        if step:
            sched.append(step)
        live = [i for i in live if at[i] < lens[i]]
    assert any(len(s) == 4 for s in sched) and any(len({c for _, c in s}) > 1 for s in sched)
    mixed = replay(eng, reqs, sched)
    st = eng.scheduler.get_stats()
    assert st["free_blocks"] == st["total_blocks"] == 11
    alone = replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i, r in enumerate(ref):
        assert within(rel_err(mixed[i], r), dtype), (i, rel_err(mixed[i], r).max())
        assert rel_err(mixed[i], alone[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else 0.2)


def test_engine_state_slots_are_handed_out_and_returned(cuda, tmp_path):
    """Each live sequence holds its own slot; a fifth is refused while four are live; a finished one's slot goes to the next
    sequence, whose state starts from zero although the slot holds the old one."""
    rng = np.random.default_rng(15)
    cfg = variant("ones")
    w = T.random_weights(cfg, rng)
    eng, _ = make_engine(tmp_path, cfg, w, "float32", bs=16, blocks=16, max_seqs=4)
    from nano_vllm_rs_b200.engine import SamplingParams
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    toks = [rng.integers(0, cfg["vocab"], 12).tolist() for _ in range(6)]
    ids = [eng.scheduler.add_sequence(t, sp) for t in toks[:5]]
    b = eng.scheduler.schedule_chunks(ids[:4], [3, 3, 3, 3])
    assert sorted(b.state_slots.tolist()) == [0, 1, 2, 3]
    eng.scheduler.commit_chunks()
    with pytest.raises(Exception):
        eng.scheduler.schedule_chunks([ids[4]], [2])
    eng.scheduler.finish_sequence(ids[1]); eng.scheduler.release_sequence(ids[1])
    for i in (0, 2, 3):
        eng.scheduler.finish_sequence(ids[i]); eng.scheduler.release_sequence(ids[i])
    first = eng.step_chunks([ids[4]], [12], list(range(12)))      # runs in a slot that others used before
    assert rel_err(first, T.logits_of(cfg, w, toks[4])).max() < TOL["float32"]


def test_engine_long_decoding_and_far_tokens(cuda, tmp_path):
    """300 tokens at once, then 60 one by one over 20+ pages: attention reads far keys through the tables, the recurrent
    states carry what the pages do not hold."""
    rng = np.random.default_rng(12)
    cfg = T.make_config([("parallel", T.parallel_mixer(**ATT, **SSD), None), ("retention", T.retention_mixer(decay=[0.999, 0.99, 0.9]), None)])
    w = T.random_weights(cfg, rng)
    toks = rng.integers(0, cfg["vocab"], 360).tolist()
    ref = T.logits_of(cfg, w, toks)
    eng, _ = make_engine(tmp_path, cfg, w, "float32", bs=16, blocks=23, max_seqs=2)
    got = replay(eng, [toks], [[(0, 300)]] + [[(0, 1)]] * 60)
    assert rel_err(got[0], ref).max() < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(cuda, tmp_path, dtype):
    """LLMEngine.generate: the scheduler's own prefill / decode batches, decode steps replayed as CUDA graphs, pages taken
    while decoding, six prompts for four state slots (two wait until a slot is free)."""
    from nano_vllm_rs_b200.engine import SamplingParams
    rng = np.random.default_rng(13)
    cfg = variant("all_kinds")
    w = T.random_weights(cfg, rng)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (5, 1, 30, 16, 3, 20)]
    n_new = 40
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=40, max_seqs=4, eager=0)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    margin_floor = 1e-3 if dtype == "float32" else 0.15
    agreed = 0
    for p, o in zip(prompts, outs):
        assert len(o) == n_new
        ref, margins = T.greedy(cfg, w, p, n_new)
        for j in range(n_new):
            if o[j] != ref[j]:
                assert margins[j] < margin_floor, (j, margins[j])   # a near-tie may fall either way; later tokens then differ
                break
            agreed += 1
    assert agreed > 0.6 * n_new * len(prompts)
    st = eng.scheduler.get_stats()
    assert st["decode_batches"] >= n_new - 1 and st["free_blocks"] == st["total_blocks"]


def test_generation_survives_preemption(cuda, tmp_path):
    """A cache pool too small for four growing sequences: the scheduler preempts (pages and state slot go back), later
    admits the victim again and recomputes it from position 0 into whatever slot is free; the tokens stay the oracle's."""
    from nano_vllm_rs_b200.engine import SamplingParams
    rng = np.random.default_rng(16)
    cfg = variant("all_kinds")
    w = T.random_weights(cfg, rng)
    prompts = [rng.integers(0, cfg["vocab"], 16).tolist() for _ in range(4)]
    n_new = 40
    eng, _ = make_engine(tmp_path, cfg, w, "float32", bs=16, blocks=11, max_seqs=4, eager=0)   # 4 x 56 tokens need 16 pages
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    st = eng.scheduler.get_stats()
    assert st["preemptions"] > 0 and st["free_blocks"] == st["total_blocks"]
    for p, o in zip(prompts, outs):
        ref, margins = T.greedy(cfg, w, p, n_new)
        for j in range(n_new):
            if o[j] != ref[j]:
                assert margins[j] < 1e-3, (j, margins[j])
                break


def test_command_line_generates_and_samples(cuda, tmp_path):
    """`python -m nano_vllm_rs_b200 generate` on a Talapel checkpoint: greedy tokens are the oracle's; with a temperature the
    device sampler draws from the same logits (tokens in range, two different prompts give different draws)."""
    import sys
    rng = np.random.default_rng(17)
    cfg = variant("all_kinds")
    w = T.random_weights(cfg, rng)
    _, model_dir = make_engine(tmp_path, cfg, w, "float32")
    prompt = rng.integers(0, cfg["vocab"], 9).tolist()
    run = lambda *extra: subprocess.run([sys.executable, "-m", "nano_vllm_rs_b200", "generate", "--model", model_dir, "--dtype", "float32",
                                         "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "12", "--block-size", "16", *extra],
                                        cwd=ROOT, capture_output=True, text=True, timeout=600)
    r = run()
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    ref, margins = T.greedy(cfg, w, prompt, 12)
    assert out["prompt_ids"] == prompt and len(out["completion_ids"]) == 12
    for j in range(12):
        if out["completion_ids"][j] != ref[j]:
            assert margins[j] < 1e-3
            break
    r = run("--temperature", "1.5", "--top-k", "20")
    assert r.returncode == 0, r.stderr[-2000:]
    sampled = json.loads(r.stdout.strip().splitlines()[-1])["completion_ids"]
    assert len(sampled) == 12 and all(0 <= t < cfg["vocab"] for t in sampled) and sampled != ref
    r = subprocess.run([sys.executable, "-m", "nano_vllm_rs_b200", "architectures"], cwd=ROOT, capture_output=True, text=True, timeout=120)
    assert "Talapel" in r.stdout


def test_trace_run_replays_a_schedule(cuda, tmp_path):
    rng = np.random.default_rng(14)
    cfg = variant("all_kinds")
    w = T.random_weights(cfg, rng)
    _, model_dir = make_engine(tmp_path, cfg, w, "float32")
    a, b = rng.integers(0, cfg["vocab"], 70).tolist(), rng.integers(0, cfg["vocab"], 9).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[:8], "want": []}, {"id": "a", "tokens": a[40:69], "want": [28]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["a", "b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    ra, rb = T.logits_of(cfg, w, a), T.logits_of(cfg, w, b)
    rd = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    for got, ref in ((rd(0), ra[[0, 39]]), (rd(1), ra[[68]]), (rd(2), np.stack([ra[69], rb[8]])), (rd(3), rb[[8]])):
        assert got.shape == ref.shape and rel_err(got, ref).max() < TOL["float32"]
