"""GPU tests of the Kosazen architecture: every mechanism's kernel against oracle/kosazen.py (plain numpy, float64), then the
engine — whole prompts, token-by-token decoding, portions down to two tokens, mixed batches, reused pages, greedy generation
through LLMEngine.generate and a replay through bin/trace_run — on small random models whose sizes are all different from
one another.  f32 engines must agree with the oracle to rounding; bf16 engines within the error of bf16 operands."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import kosazen as K

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def dev_t(a, dev, dtype):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).to(dtype)


def rel_err(got, ref):
    """Per row: rms of the centred difference over the rms of the centred reference."""
    d = np.asarray(got, np.float64) - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((r ** 2).mean(-1))


# ------------------------------------------------------------------------------------------------ mechanisms alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dyt_residual_norm(cuda, dtype):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(1)
    n, hid = 37, 50
    h = rng.standard_normal((n, hid)) * 3
    y = K.bf16_round(rng.standard_normal((n, hid)))
    w = {k: rng.standard_normal(hid) for k in ("a", "a.b", "c", "c.b")}
    w["a.alpha"], w["c.alpha"] = 0.7, 1.4
    par = lambda k: (dev_t([w[k + ".alpha"]], cuda, torch.float32), dev_t(w[k], cuda, torch.float32), dev_t(w[k + ".b"], cuda, torch.float32))
    hd = dev_t(h, cuda, torch.float32)
    out = ops.dyt_residual_norm(hd, dev_t(y, cuda, dtype), post=par("a"), pre=par("c"), dtype=dtype)
    h_ref = h.astype(np.float32).astype(np.float64) + K.dyt(y, w, "a")
    np.testing.assert_allclose(hd.cpu().numpy(), h_ref, rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(out.float().cpu().numpy(), K.dyt(h_ref, w, "c"), rtol=1e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-5)
    only = ops.dyt_residual_norm(hd, None, pre=par("c"), dtype=dtype)   # input norm alone leaves h untouched
    assert torch.equal(only, out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(37, 45, 51), (1, 7, 3), (130, 136, 128), (5, 64, 192), (300, 8, 64)])
def test_linear_any_sizes(cuda, dtype, m, n, k):
    """Odd sizes run on the tile kernel, (k % 64, n % 8) bf16 shapes on the tensor-core GEMM: both against float64."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(m * 1000 + n)
    x, w = K.bf16_round(rng.standard_normal((m, k))), K.bf16_round(rng.standard_normal((n, k)) / np.sqrt(k))
    y = ops.linear(dev_t(x, cuda, dtype), dev_t(w, cuda, dtype), out_dtype=torch.float32)
    np.testing.assert_allclose(y.cpu().numpy(), x @ w.T, rtol=1e-4, atol=2e-5)
    if dtype == torch.bfloat16:
        yb = ops.linear(dev_t(x, cuda, dtype), dev_t(w, cuda, dtype))
        np.testing.assert_allclose(yb.float().cpu().numpy(), x @ w.T, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_batched_per_head_views(cuda, dtype):
    """Per-head projection out of a packed activation: x[t, h, :dim] (row stride = whole packed row) times w[h]."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(3)
    T, H, dim, extra, r = 19, 3, 12, 6, 20
    packed = K.bf16_round(rng.standard_normal((T, H * (dim + extra) + 11)))
    w = K.bf16_round(rng.standard_normal((H, r, dim)))
    xd = dev_t(packed, cuda, dtype)
    out = torch.zeros((T, H * r), dtype=torch.float32, device=cuda)
    ops.linear(xd, dev_t(w.reshape(H * r, dim), cuda, dtype), out_dtype=torch.float32, batch=H, bsx=dim + extra, bsw=r * dim, bsy=r,
               out=out, n=r, k=dim)
    ref = np.stack([packed[:, h * (dim + extra):h * (dim + extra) + dim] @ w[h].T for h in range(H)], 1).reshape(T, H * r)
    np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=1e-5, atol=1e-5)


def test_rope_table_and_latent_prepare(cuda):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(4)
    T, H, dim, rd, r, dims, base, eps = 9, 3, 10, 8, 14, 6, 777.0, 1e-5   # dims < rot_dim: the tail passes unchanged
    pos = np.array([0, 1, 2, 63, 64, 65, 500, 1999, 7])
    tab = ops.rope_table_interleaved(2000, dims, base, cuda).cpu().numpy()
    for p in (1, 65, 1999):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            np.testing.assert_allclose(tab[p, i], [np.cos(a), np.sin(a)], atol=1e-6)
    q = rng.standard_normal((T, H * (dim + rd)))
    dkv = rng.standard_normal((T, r + rd))
    g = rng.standard_normal(r)
    slots = np.array([5, 0, 17, 3, -1, 8, 9, 10, 11], np.int32)
    cache = torch.zeros((20, r + rd + 2), dtype=torch.float32, device=cuda)
    qd = dev_t(q, cuda, torch.float32)
    ops.latent_prepare(qd, dev_t(dkv, cuda, torch.float32), dev_t(g, cuda, torch.float32), eps, torch.from_numpy(pos).to(cuda),
                       ops.rope_table_interleaved(2000, dims, base, cuda), dims, H, dim, rd, r, cache, torch.from_numpy(slots).to(cuda))
    got_q, got_c = qd.cpu().numpy().reshape(T, H, dim + rd), cache.cpu().numpy()
    for t in range(T):
        c_ref = K.rms_norm(dkv[t, :r].astype(np.float32).astype(np.float64), g.astype(np.float32), eps)
        kr_ref = K.rotate_pairs(dkv[t, r:], pos[t], dims, base)
        if slots[t] >= 0:
            np.testing.assert_allclose(got_c[slots[t], :r], c_ref, rtol=1e-5, atol=1e-5)
            np.testing.assert_allclose(got_c[slots[t], r:r + rd], kr_ref, rtol=1e-5, atol=2e-5)
        for h in range(H):
            qh = q[t].reshape(H, dim + rd)[h]
            np.testing.assert_allclose(got_q[t, h, :dim], qh[:dim], rtol=1e-6)
            np.testing.assert_allclose(got_q[t, h, dim:], K.rotate_pairs(qh[dim:], pos[t], dims, base), rtol=1e-5, atol=2e-5)
    assert np.all(got_c[4] == 0) and np.all(got_c[:, r + rd:] == 0)   # slot -1 stored nothing; padding untouched


def _attention_ref(q_abs, q_rot, rows, scale, r):
    s = np.array([(q_abs @ row[:r] + q_rot @ row[r:]) * scale for row in rows])
    e = np.exp(s - s.max())
    p = e / e.sum()
    return (p[:, None] * np.stack(rows)[:, :r]).sum(0), p


def _paged_case(rng, ctx, bs, row, extra=3):
    """Random cache rows for sequences of the given lengths behind shuffled block tables."""
    nblk = [(c + bs - 1) // bs for c in ctx]
    ids = rng.permutation(sum(nblk) + extra)
    cache = rng.standard_normal((len(ids) * bs, row))   # unwritten slots hold noise, never zeros
    tables = np.full((len(ctx), max(nblk) + 1), -1, np.int32)
    seqs, k = [], 0
    for b, c in enumerate(ctx):
        rows = rng.standard_normal((c, row))
        for j in range(nblk[b]):
            tables[b, j] = ids[k]; k += 1
            n = min(bs, c - j * bs)
            cache[tables[b, j] * bs: tables[b, j] * bs + n] = rows[j * bs: j * bs + n]
        seqs.append(rows)
    return cache, tables, seqs


@pytest.mark.parametrize("H", [5, 19])   # 19 heads: more than one head group per token in both kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_paged_positions(cuda, dtype, H):
    """Queries at the first positions, just before / at / after page borders and deep into long sequences; several query
    tokens of one sequence in one launch (a prompt portion) beside single tokens of others."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(5)
    dim, rd, r, bs, scale = 9, 6, 40, 16, 0.21
    ctx = [1, 15, 16, 17, 33, 150, 331]
    cache, tables, seqs = _paged_case(rng, ctx, bs, r + rd)
    if dtype == torch.bfloat16:
        cache, seqs = K.bf16_round(cache), [K.bf16_round(s) for s in seqs]
    tok_seq, pos = [], []
    for b, c in enumerate(ctx):
        for p in sorted({0, c - 1, max(0, c - 2), min(c - 1, 15), min(c - 1, 16), c // 2}):
            tok_seq.append(b); pos.append(p)
    n = len(pos)
    q_abs = rng.standard_normal((n, H, r))
    q = K.bf16_round(rng.standard_normal((n, H, dim + rd)))
    out = ops.latent_attention(dev_t(q_abs.reshape(n, -1), cuda, torch.float32), dev_t(q.reshape(n, -1), cuda, dtype),
                               torch.tensor(tok_seq, dtype=torch.int32, device=cuda), torch.tensor(pos, dtype=torch.int64, device=cuda),
                               torch.from_numpy(tables).to(cuda), bs, dev_t(cache, cuda, dtype), H, dim, rd, r, scale)
    got = out.float().cpu().numpy().reshape(n, H, r)
    qa32 = q_abs.astype(np.float32).astype(np.float64)
    for i in range(n):
        rows = list(seqs[tok_seq[i]][:pos[i] + 1])
        for h in range(H):
            ref, _ = _attention_ref(qa32[i, h], q[i, h, dim:], rows, scale, r)
            np.testing.assert_allclose(got[i, h], ref, rtol=2e-2 if dtype == torch.bfloat16 else 1e-4, atol=2e-2 if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("where", ["first", "far", "page_end", "page_start", "last", "next"])
def test_latent_attention_one_key_stands_out(cuda, where, dtype):
    """One cached row is made to dominate the scores: the output must be that row's latent when it is visible (the first
    token, a key hundreds back, a page's last / first slot, the query's own row) and must not show it when it lies one
    position in the future."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(6)
    H, dim, rd, r, bs, scale = 2, 4, 4, 24, 16, 1.0
    ctx, qpos = 420, 400
    target = {"first": 0, "far": 37, "page_end": 16 * 20 - 1, "page_start": 16 * 20, "last": qpos, "next": qpos + 1}[where]
    cache, tables, seqs = _paged_case(rng, [ctx], bs, r + rd)
    rows = K.bf16_round(seqs[0] * 0.05)
    rows[target, r:] = 6.0                       # its rotated key part lines up with the query's
    blk, off = tables[0, target // bs], target % bs
    for j in range(ctx):
        cache[tables[0, j // bs] * bs + j % bs] = rows[j]
    q = np.zeros((1, H, dim + rd)); q[0, :, dim:] = 6.0
    q_abs = np.zeros((1, H * r))
    out = ops.latent_attention(dev_t(q_abs, cuda, torch.float32), dev_t(q.reshape(1, -1), cuda, dtype),
                               torch.zeros(1, dtype=torch.int32, device=cuda), torch.tensor([qpos], dtype=torch.int64, device=cuda),
                               torch.from_numpy(tables).to(cuda), bs, dev_t(cache, cuda, dtype), H, dim, rd, r, scale)
    got = out.float().cpu().numpy().reshape(H, r)
    tol = 1e-5 if dtype == torch.float32 else 2e-3
    assert cache[blk * bs + off, r] == 6.0
    if where == "next":
        ref, _ = _attention_ref(np.zeros(r), q[0, 0, dim:], list(rows[:qpos + 1]), scale, r)
        np.testing.assert_allclose(got[0], ref, rtol=1e-4, atol=tol)
        assert np.abs(got[0] - rows[target, :r]).max() > 0.01
    else:
        np.testing.assert_allclose(got[0], rows[target, :r], atol=tol)   # exp(-(144 - small)) leaves nothing of the others


def test_moe_route_sort_grouped_combine(cuda):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(7)
    n, W, E, I, top, ff, lim, rs = 70, 24, 5, 3, 3, 20, 0.8, 1.7
    w = {"router": rng.standard_normal((E + I, W)), "correction": np.array([0.5, -0.5, 0, 0, 0.3, -0.2, 0.4, 0.0])}
    for e in range(E):
        w["e%d.gate" % e], w["e%d.up" % e] = rng.standard_normal((ff, W)), rng.standard_normal((ff, W))
        w["e%d.down" % e] = rng.standard_normal((W, ff)) / 4
    w = {k: v.astype(np.float32).astype(np.float64) for k, v in w.items()}
    x = rng.standard_normal((n, W)).astype(np.float32).astype(np.float64) / 3
    f32 = torch.float32
    xd = dev_t(x, cuda, f32)
    logits = ops.linear(xd, dev_t(w["router"], cuda, f32), out_dtype=f32)
    idx, wt = ops.moe_route(logits, dev_t(w["correction"], cuda, f32), top, rs)
    r = {"experts": E, "identity": I, "top": top, "scale": rs}
    chosen = 0
    for t in range(n):
        ri, rw, margin = K.route(x[t], w, "", r)
        if margin > 1e-5:
            assert sorted(idx[t].tolist()) == sorted(ri.tolist()), t
            got = dict(zip(idx[t].tolist(), wt[t].tolist()))
            np.testing.assert_allclose([got[i] for i in ri], rw, rtol=1e-5)
            chosen += 1
    assert chosen > n * 0.9 and (idx >= E).any() and (idx < E).any()
    row_token, tile_expert, slot_row = ops.moe_sort(idx, E)
    rt, te, sr = row_token.cpu().numpy(), tile_expert.cpu().numpy(), slot_row.cpu().numpy()
    for t in range(n):
        for k in range(top):
            e = int(idx[t, k])
            if e >= E:
                assert sr[t, k] == -1
            else:
                assert rt[sr[t, k]] == t and te[sr[t, k] // 32] == e
    assert (rt >= 0).sum() == int((idx < E).sum())
    egu = np.stack([np.concatenate([w["e%d.gate" % e], w["e%d.up" % e]]) for e in range(E)])
    edown = np.stack([w["e%d.down" % e] for e in range(E)])
    act = ops.linear_grouped(xd, dev_t(egu, cuda, f32), row_token, tile_expert, rt.size, ff, W, 2 * ff * W, glu=True, limit=lim)
    eout = ops.linear_grouped(act, dev_t(edown, cuda, f32), None, tile_expert, rt.size, W, ff, W * ff)
    shared = dev_t(rng.standard_normal((n, W)), cuda, f32)
    out = ops.moe_combine(eout, xd, shared, idx, wt, slot_row, E).cpu().numpy()
    idx_h, wt_h = idx.cpu().numpy(), wt.cpu().numpy()
    for t in range(n):
        ref = shared[t].cpu().numpy().astype(np.float64)
        for k in range(top):
            e = idx_h[t, k]
            ref = ref + wt_h[t, k] * (K.glu_expert(x[t], w["e%d.gate" % e], w["e%d.up" % e], w["e%d.down" % e], lim) if e < E else x[t])
        np.testing.assert_allclose(out[t], ref, rtol=1e-4, atol=1e-5)
    g = ops.glu_clamped(dev_t(np.concatenate([x @ w["e0.gate"].T, x @ w["e0.up"].T], 1), cuda, f32), lim).cpu().numpy()
    gg, uu = np.minimum(x @ w["e0.gate"].T, lim), np.clip(x @ w["e0.up"].T, -lim, lim)
    np.testing.assert_allclose(g, gg / (1 + np.exp(-1.702 * gg)) * (uu + 1), rtol=1e-5, atol=1e-6)


def test_moe_route_top1_and_bias_decides(cuda):
    """top = 1; a selection bias changes WHICH expert is chosen but not the weight, which comes from the unbiased score."""
    from nano_vllm_rs_b200 import ops
    z = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device=cuda)
    idx, w = ops.moe_route(z, None, 1, 2.5)
    assert idx.item() == 0 and abs(w.item() - 2.5) < 1e-6          # one chosen: s / s * scale
    idx, w = ops.moe_route(z, torch.tensor([0.0, 0.0, 0.0, 0.9], device=cuda), 2, 1.0)
    s = np.exp([2.0, 1, 0, -1]); s /= s.sum()
    assert sorted(idx[0].tolist()) == [0, 3]
    got = dict(zip(idx[0].tolist(), w[0].tolist()))
    np.testing.assert_allclose([got[0], got[3]], [s[0] / (s[0] + s[3]), s[3] / (s[0] + s[3])], rtol=1e-5)


# ------------------------------------------------------------------------------------------------ the engine


VARIANTS = {
    # every size different from every other; a looped range; identity experts; three of seven router outputs chosen
    "odd_looped": dict(n_layers=3, loop=(1, 2, 3)),
    # sizes the tensor-core GEMM takes (k % 64, n % 8); a layer without feed-forward; no identity experts, no shared expert, top 1
    "aligned_plain": dict(vocab=128, width=64, n_layers=3, mlp_mask=[1, 0, 1], heads=2, dim=32, rot_dim=8, vdim=32, kv_rank=24,
                          ff=64, experts=4, identity=0, top=1, shared=False, router_scale=1.0),
    # nothing divisible by 8, 4 or 2 except the rotated pairs; odd vocabulary
    "primes": dict(vocab=101, width=37, n_layers=2, heads=3, dim=7, rot_dim=4, vdim=5, kv_rank=11, ff=13, shared_ff=9, experts=3,
                   identity=1, top=2),
    # one head, one real expert, every router output chosen, loop that covers everything once
    "ones": dict(n_layers=2, loop=(0, 2, 1), heads=1, dim=8, rot_dim=8, vdim=8, kv_rank=8, experts=1, identity=1, top=2, ff=8, shared_ff=8, width=8),
}


def make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=24, max_seqs=4, eager=1):
    from nano_vllm_rs_b200.engine import LLMEngine
    from nano_vllm_rs_b200.loader import write_safetensors
    d = tmp_path / ("m_" + dtype)
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: K.to_bf16_bits(v) for k, v in w.items()})
    return LLMEngine.from_pretrained(str(d), dtype=dtype, kvcache_block_size=bs, num_kvcache_blocks=blocks, max_num_seqs=max_seqs,
                                     max_num_batched_tokens=blocks * bs, max_model_len=blocks * bs, enforce_eager=eager), str(d)


def replay(eng, requests, schedule):
    """schedule: steps of [(request index, token count)].  Returns per request the logits of ALL its positions."""
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


def oracle_logits(cfg, w, reqs, dtype):
    """Oracle logits per request and, per request, the positions that are compared: all of them in f32; in bf16 those whose
    routers all chose with a clear margin (where two selection scores nearly tie, bf16 operands may pick the other expert —
    a different, equally valid function value, not an error of a kernel)."""
    ref, sure = [], []
    for r in reqs:
        m = []
        ref.append(K.logits_of(cfg, w, r, m))
        sure.append(np.asarray(m) > (0.0 if dtype == "float32" else 0.003))
    assert np.concatenate(sure).mean() > 0.6
    return ref, sure


def cut(n, sizes):
    out, k = [], 0
    while n > 0:
        c = min(n, sizes[k % len(sizes)]); out.append(c); n -= c; k += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", list(VARIANTS))
def test_engine_schedules_match_the_oracle(cuda, tmp_path, variant, dtype):
    rng = np.random.default_rng(100 + list(VARIANTS).index(variant))
    cfg = K.random_config(rng, **VARIANTS[variant])
    w = K.random_weights(cfg, rng)
    lens = [1, 2, 37, 70, 33]
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in lens]
    ref, sure = oracle_logits(cfg, w, reqs, dtype)
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=12)    # 192 slots: the requests only fit one after another
    tol = TOL[dtype]

    def check(got, what):
        for i, r in enumerate(ref):
            e = rel_err(got[i], r)
            assert np.isfinite(e).all() and (e[sure[i]].max() if sure[i].any() else 0.0) < tol, \
                f"{variant} {dtype} {what}: request {i} position {int(e.argmax())} error {e.max():.3g}"

    whole = replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    check(whole, "whole prompts")
    # most of the prompt at once, the last tokens one by one (decoding through the cache across page borders)
    dec = replay(eng, reqs, [s for i, r in enumerate(reqs) for s in ([[(i, max(1, len(r) - 20))]] + [[(i, 1)]] * (len(r) - max(1, len(r) - 20)))])
    check(dec, "prefill + single tokens")
    # everything token by token
    one = replay(eng, reqs[:3], [[(i, 1)] for i, r in enumerate(reqs[:3]) for _ in r])
    for i in range(3):
        assert not sure[i].any() or rel_err(one[i], ref[i])[sure[i]].max() < tol
    # portions of changing size down to two tokens
    por = replay(eng, reqs, [[(i, c)] for i, r in enumerate(reqs) for c in cut(len(r), [2, 5, 16, 3, 17, 2, 31])])
    check(por, "portions")
    # the same position must not depend on how the prompt was cut, beyond rounding
    for i in range(len(reqs)):
        assert rel_err(por[i], whole[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_mixed_batches_and_reused_pages(cuda, tmp_path, dtype):
    """Up to four live requests per step, portions of some beside single tokens of others, in a pool that only holds them
    because finished requests give their pages back; every request equals its run alone and the oracle."""
    rng = np.random.default_rng(11)
    cfg = K.random_config(rng, n_layers=2, loop=(0, 1, 2))
    w = K.random_weights(cfg, rng)
    lens = [50, 23, 64, 9, 41, 30, 17]
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in lens]
    ref, sure = oracle_logits(cfg, w, reqs, dtype)
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=11, max_seqs=4)   # 176 slots < 234 tokens in total
    need = [(n + 15) // 16 for n in lens]            # pages a request holds by its end; admitted only when they are free
    at, live, nxt, sched, k = [0] * len(lens), [], 0, [], 0
    while nxt < len(reqs) or live:
        while nxt < len(reqs) and len(live) < 4 and sum(need[i] for i in live) + need[nxt] <= 11:
            live.append(nxt); nxt += 1
        step = []
        for i in live:
            k += 1
            c = 1 if (at[i] > lens[i] // 2 or k % 3 == 0) else [2, 7, 16, 5][k % 4]
            c = min(c, lens[i] - at[i])
            step.append((i, c)); at[i] += c
        sched.append(step)
        live = [i for i in live if at[i] < lens[i]]
    assert any(len(s) == 4 for s in sched) and any(len({c for _, c in s}) > 1 for s in sched)
    mixed = replay(eng, reqs, sched)
    st = eng.scheduler.get_stats()
    assert st["free_blocks"] == st["total_blocks"] == 11
    alone = replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i, r in enumerate(ref):
        assert not sure[i].any() or rel_err(mixed[i], r)[sure[i]].max() < TOL[dtype], (i, rel_err(mixed[i], r).max())
        assert rel_err(mixed[i], alone[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else TOL[dtype])


def test_engine_far_keys_over_many_pages(cuda, tmp_path):
    """A few hundred tokens in one sequence (20+ pages), read back token by token at the end."""
    rng = np.random.default_rng(12)
    cfg = K.random_config(rng, n_layers=1, mlp_mask=[0], heads=2, scale=0.6)
    w = K.random_weights(cfg, rng)
    toks = rng.integers(0, cfg["vocab"], 340).tolist()
    ref = K.logits_of(cfg, w, toks)
    eng, _ = make_engine(tmp_path, cfg, w, "float32", bs=16, blocks=22, max_seqs=2)
    got = replay(eng, [toks], [[(0, 300)]] + [[(0, 1)]] * 40)
    assert rel_err(got[0], ref).max() < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(cuda, tmp_path, dtype):
    """LLMEngine.generate: the scheduler's own prefill / decode batches, decode steps replayed as CUDA graphs, pages taken
    while decoding (block size 16, 40 new tokens), unequal prompts in one batch."""
    from nano_vllm_rs_b200.engine import SamplingParams
    rng = np.random.default_rng(13)
    cfg = K.random_config(rng, n_layers=2, loop=(1, 2, 2))
    w = K.random_weights(cfg, rng)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (5, 1, 30, 16)]
    n_new = 40
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=40, max_seqs=4, eager=0)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    margin_floor = 1e-3 if dtype == "float32" else 0.15
    agreed = 0
    for p, o in zip(prompts, outs):
        assert len(o) == n_new
        ref, margins = K.greedy(cfg, w, p, n_new)
        for j in range(n_new):
            if o[j] != ref[j]:
                assert margins[j] < margin_floor, (j, margins[j])   # a near-tie may fall either way; later tokens then differ
                break
            agreed += 1
    assert agreed > 0.6 * n_new * len(prompts)
    st = eng.scheduler.get_stats()
    assert st["decode_batches"] >= n_new - 1 and st["free_blocks"] == st["total_blocks"]


def test_trace_run_replays_a_schedule(cuda, tmp_path):
    rng = np.random.default_rng(14)
    cfg = K.random_config(rng, n_layers=2)
    w = K.random_weights(cfg, rng)
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
    ra, rb = K.logits_of(cfg, w, a), K.logits_of(cfg, w, b)
    rd = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    for got, ref in ((rd(0), ra[[0, 39]]), (rd(1), ra[[68]]), (rd(2), np.stack([ra[69], rb[8]])), (rd(3), rb[[8]])):
        assert got.shape == ref.shape and rel_err(got, ref).max() < TOL["float32"]


def test_grouped_tensor_core_gemm(cuda):
    """128-row tiles, each against its own expert's weight block; unused tiles and padding rows are never read back."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(15)
    n_tok, W, E, top, ff = 300, 128, 5, 2, 192
    idx = torch.from_numpy(np.stack([rng.permutation(E + 1)[:top] for _ in range(n_tok)]).astype(np.int32)).to(cuda)   # E = identity
    row_token, tile_expert, slot_row = ops.moe_sort(idx, E, tile_rows=128)
    rt, te, sr = row_token.cpu().numpy(), tile_expert.cpu().numpy(), slot_row.cpu().numpy()
    assert rt.size % 128 == 0 and te.size == rt.size // 128 and (te >= 0).sum() >= E
    x = K.bf16_round(rng.standard_normal((n_tok, W)))
    w = K.bf16_round(rng.standard_normal((E, ff, W)) / np.sqrt(W))
    xg = torch.zeros((rt.size, W), dtype=torch.bfloat16, device=cuda)
    xg[torch.from_numpy(rt >= 0).to(cuda)] = dev_t(x[rt[rt >= 0]], cuda, torch.bfloat16)
    y = ops.gemm_bf16_grouped(xg, dev_t(w.reshape(E * ff, W), cuda, torch.bfloat16), tile_expert, ff, E).float().cpu().numpy()
    idx_h = idx.cpu().numpy()
    for t in range(0, n_tok, 7):
        for k in range(top):
            e = idx_h[t, k]
            if e < E:
                assert te[sr[t, k] // 128] == e
                np.testing.assert_allclose(y[sr[t, k]], x[t] @ w[e].T, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_whole_prompts_in_one_launch(cuda, dtype):
    """Every position of several sequences as a query in ONE launch of more than 256 tokens (the bf16 kernel then takes two
    neighbouring tokens per CTA): odd and even lengths and a one-token sequence, so that pairs fall inside a sequence, on a
    sequence's last token and across two sequences."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(16)
    H, dim, rd, r, bs, scale = 3, 8, 6, 40, 16, 0.3
    ctx = [5, 130, 131, 64, 1, 77]
    cache, tables, seqs = _paged_case(rng, ctx, bs, r + rd)
    if dtype == torch.bfloat16:
        cache, seqs = K.bf16_round(cache), [K.bf16_round(s) for s in seqs]
    tok_seq = np.concatenate([np.full(c, b) for b, c in enumerate(ctx)]).astype(np.int32)
    pos = np.concatenate([np.arange(c) for c in ctx]).astype(np.int64)
    n = len(pos)
    assert n > 256
    q_abs = rng.standard_normal((n, H, r)).astype(np.float32)
    q = K.bf16_round(rng.standard_normal((n, H, dim + rd)))
    out = ops.latent_attention(dev_t(q_abs.reshape(n, -1), cuda, torch.float32), dev_t(q.reshape(n, -1), cuda, dtype),
                               torch.from_numpy(tok_seq).to(cuda), torch.from_numpy(pos).to(cuda), torch.from_numpy(tables).to(cuda),
                               bs, dev_t(cache, cuda, dtype), H, dim, rd, r, scale)
    got = out.float().cpu().numpy().reshape(n, H, r)
    qa = K.bf16_round(q_abs) if dtype == torch.bfloat16 else q_abs.astype(np.float64)   # the bf16 kernel rounds the folded query
    t0 = 0
    for b, c in enumerate(ctx):
        rows = seqs[b]
        for h in range(H):
            s = (qa[t0:t0 + c, h] @ rows[:, :r].T + q[t0:t0 + c, h, dim:] @ rows[:, r:].T) * scale
            s = np.where(np.tril(np.ones((c, c), bool)), s, -np.inf)
            p = np.exp(s - s.max(-1, keepdims=True))
            ref = (p / p.sum(-1, keepdims=True)) @ rows[:, :r]
            np.testing.assert_allclose(got[t0:t0 + c, h], ref, rtol=2e-2 if dtype == torch.bfloat16 else 1e-4,
                                       atol=2e-2 if dtype == torch.bfloat16 else 1e-5)
        t0 += c


def test_long_prompt_takes_the_per_head_gemm_path(cuda, tmp_path):
    """A bf16 prompt of more than 512 tokens with tensor-core sizes: the per-head projections run as one GEMM per head on
    views of the packed activations, attention takes two tokens per CTA; then single tokens continue from that cache."""
    rng = np.random.default_rng(17)
    cfg = K.random_config(rng, vocab=64, width=64, n_layers=1, mlp_mask=[0], heads=2, dim=64, rot_dim=8, vdim=16, kv_rank=64, scale=0.12)
    w = K.random_weights(cfg, rng)
    toks = rng.integers(0, cfg["vocab"], 536).tolist()
    ref = K.logits_of(cfg, w, toks)
    eng, _ = make_engine(tmp_path, cfg, w, "bfloat16", bs=16, blocks=36, max_seqs=2)
    got = replay(eng, [toks], [[(0, 530)]] + [[(0, 1)]] * 6)
    assert rel_err(got[0], ref).max() < TOL["bfloat16"]
