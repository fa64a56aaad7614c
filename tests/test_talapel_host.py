"""CPU tests around the Talapel integration: properties of the oracle's mechanisms that hold by construction, the model
registry's configuration reader, and the scheduler's pool of recurrent-state slots (explicit stepping and the regular
prefill / decode schedule: admission, refusal, reuse, no prefix sharing)."""
import json

import numpy as np
import pytest

from oracle import talapel as T


def small_cfg(**kw):
    return T.make_config([("parallel", T.parallel_mixer(), T.dense_mlp(10)), ("retention", T.retention_mixer(), T.expert_mlp()),
                          ("retention", T.retention_mixer(heads=2, dim=6, vdim=5, rot_dims=6), None)], **kw)


# ------------------------------------------------------------------------------------------------ oracle properties


def test_retention_equals_its_unrolled_sum():
    """o_t = sum_{j <= t} decay^(t-j) (q_t . k_j) v_j before the norm: the recurrence and the explicit sum agree."""
    rng = np.random.default_rng(0)
    m = T.retention_mixer(heads=2, dim=6, vdim=4, rot_dims=4, rot_base=50.0, decay=[0.9, 0.5])
    W, eps = 10, 1e-5
    w = {k: rng.standard_normal(s) for k, s in (("q", (12, W)), ("k", (12, W)), ("v", (8, W)), ("g", (8, W)))}
    w["o"] = np.eye(8)
    hs = rng.standard_normal((7, W))
    S = np.zeros((2, 6, 4))
    outs = [T.retention_token(h, w, "", m, eps, t, S) for t, h in enumerate(hs)]
    t = 6
    q = T.rotate_half((w["q"] @ hs[t]).reshape(2, 6), t, 4, 50.0)
    for hh in range(2):
        o = np.zeros(4)
        for j in range(t + 1):
            k = T.rotate_half((w["k"] @ hs[j]).reshape(2, 6), j, 4, 50.0)[hh] * 6 ** -0.5
            o += m["decay"][hh] ** (t - j) * (q[hh] @ k) * (w["v"] @ hs[j]).reshape(2, 4)[hh]
        ref = T.rms(o, eps) * T.silu(w["g"] @ hs[t]).reshape(2, 4)[hh]
        np.testing.assert_allclose(outs[t].reshape(2, 4)[hh], ref, rtol=1e-10)


def test_rotation_depends_on_distance_only_and_leaves_the_tail():
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal((1, 10)), rng.standard_normal((1, 10))
    d = lambda pq, pk: (T.rotate_half(q, pq, 6, 300.0) @ T.rotate_half(k, pk, 6, 300.0).T).item()
    assert abs(d(17, 5) - d(112, 100)) < 1e-9 and abs(d(17, 5) - d(17, 6)) > 1e-6
    assert np.allclose(T.rotate_half(q, 9, 6, 300.0)[:, 6:], q[:, 6:]) and np.allclose(T.rotate_half(q, 0, 6, 300.0), q)
    r = T.rotate_half(q, 3, 6, 300.0)                       # dimension 0 pairs with dimension 3, not with its neighbour
    a = 3.0
    np.testing.assert_allclose([r[0, 0], r[0, 3]], [q[0, 0] * np.cos(a) - q[0, 3] * np.sin(a), q[0, 3] * np.cos(a) + q[0, 0] * np.sin(a)])


def test_query_temperature_steps():
    t = [T.query_temperature(p, 0.5, 4) for p in range(9)]
    assert t[0] == t[2] == 1.0 and t[3] == t[6] == 1.0 + 0.5 * np.log(2.0) and t[7] == 1.0 + 0.5 * np.log(3.0)


def test_ssd_window_and_state():
    """The convolution sees zeros before the start and exactly `taps` tokens; a token's effect on later ones goes through S."""
    rng = np.random.default_rng(2)
    m = T.parallel_mixer(s_heads=2, groups=1, state=3, s_vdim=2, taps=3, norm_groups=2)["right"]
    cfg = T.make_config([("parallel", T.parallel_mixer(s_heads=2, groups=1, state=3, s_vdim=2, taps=3, norm_groups=2), None)], width=8)
    w = {k[len("l0.mix.right."):]: v for k, v in T.random_weights(cfg, rng).items() if k.startswith("l0.mix.right.")}
    hs = rng.standard_normal((6, 8))
    st = T.SsdState(m)
    full = [T.ssd_token(h, w, "", m, 1e-5, st) for h in hs]
    assert st.window.shape == (2, 2 * 2 + 2 * 3) and np.allclose(st.window[-1], (w["in"] @ hs[-1])[4:4 + 10])
    st2 = T.SsdState(m)
    hs2 = hs.copy(); hs2[0] += 1.0                            # a change at token 0 reaches token 5 (three taps cannot): through S
    alt = [T.ssd_token(h, w, "", m, 1e-5, st2) for h in hs2]
    assert np.abs(alt[5] - full[5]).max() > 1e-9


def test_loop_order_and_first_of_pass():
    cfg = small_cfg(loop=(1, 3, 2))
    assert T.layer_runs(cfg) == [(0, False), (1, True), (2, False), (1, True), (2, False)]
    assert T.layer_runs(small_cfg()) == [(0, False), (1, False), (2, False)]
    assert "loop.in" in T.tensor_shapes(cfg) and "loop.in" not in T.tensor_shapes(small_cfg())
    assert len(T.Sequence(cfg).state) == 5


def test_table_experts_average_the_named_experts():
    rng = np.random.default_rng(3)
    f = T.expert_mlp(3, 2, 4)
    w = {"table": np.array([[2, 0], [1, 2]], np.int32)}
    for e in range(3):
        w["e%d.up" % e], w["e%d.down" % e] = rng.standard_normal((4, 5)), rng.standard_normal((5, 4))
    h = rng.standard_normal(5)
    one = lambda e: w["e%d.down" % e] @ np.maximum(w["e%d.up" % e] @ h, 0) ** 2
    np.testing.assert_allclose(T.table_experts(h, w, "", f, 1), (one(1) + one(2)) / 2)


# ------------------------------------------------------------------------------------------------ registry / configuration


def test_model_registry_reads_config_json():
    from nano_vllm_rs_b200.engine import Config, lib
    assert b"Talapel" in lib().nvllm_registered_architectures()
    c = Config(model_config=json.dumps(small_cfg(loop=(0, 2, 3), vocab=77, width=24)))
    assert (c.arch, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Talapel", 77, 24, 7)   # layer RUNS: 3 x 2 + 1
    assert c.recurrent_state == 1
    assert Config("tiny").recurrent_state == 0


@pytest.mark.parametrize("breakage,needle", [
    (lambda c: c["layers"][0].update(type="windowed"), "windowed"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "attention"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=5), "state-space"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=99), "experts"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "sparse"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
])
def test_bad_model_configs_are_refused_with_a_reason(breakage, needle):
    from nano_vllm_rs_b200 import _ffi
    from nano_vllm_rs_b200.engine import Config
    cfg = small_cfg()
    breakage(cfg)
    with pytest.raises(_ffi.NvllmError) as e:
        Config(model_config=json.dumps(cfg))
    assert needle in str(e.value)


def test_loader_passes_integer_tables_through(tmp_path):
    from nano_vllm_rs_b200.loader import ModelLoader, write_safetensors

    class Sink:
        def __init__(self): self.got = {}
        def load_weight(self, name, bits): self.got[name] = bits

    tab = np.array([[1, 0], [2, 1], [0, 2]], np.int32)
    write_safetensors(str(tmp_path / "m.safetensors"), {"l0.mlp.table": tab, "v": T.to_bf16_bits(np.ones(3))})
    sink = Sink()
    assert ModelLoader(sink).load_safetensors(str(tmp_path / "m.safetensors")) == 2
    assert sink.got["l0.mlp.table"].dtype == np.int32 and np.array_equal(sink.got["l0.mlp.table"], tab) and sink.got["v"].dtype == np.uint16


# ------------------------------------------------------------------------------------------------ state slots


def stateful_sched(blocks=8, bs=16, seqs=3, batched=64):
    from nano_vllm_rs_b200.engine import Config, Scheduler
    cfg = Config(model_config=json.dumps(small_cfg()), kvcache_block_size=bs, num_kvcache_blocks=blocks, max_num_seqs=seqs,
                 max_num_batched_tokens=batched, max_model_len=blocks * bs)
    return Scheduler(cfg)


def test_portion_steps_hand_out_slots_lowest_first_and_take_them_back():
    from nano_vllm_rs_b200 import _ffi
    from nano_vllm_rs_b200.engine import SamplingParams
    s = stateful_sched()
    sp = SamplingParams(temperature=0.0, max_tokens=1)
    ids = [s.add_sequence(list(range(5 + i)), sp) for i in range(4)]
    b = s.schedule_chunks([ids[2], ids[0]], [2, 5])
    assert b.state_slots.tolist() == [0, 1]
    s.commit_chunks()
    with pytest.raises(_ffi.NvllmError):
        s.schedule_chunks([ids[0]], [1])                       # sequence 0 has no token left
    b = s.schedule_chunks([ids[1], ids[2]], [3, 1])
    assert b.state_slots.tolist() == [2, 0]                    # a sequence keeps its slot from step to step
    s.commit_chunks()
    with pytest.raises(_ffi.NvllmError) as e:
        s.schedule_chunks([ids[3]], [2])                       # three slots, three holders
    assert "state slot" in str(e.value) and s.get_stats()["waiting"] == 1
    s.finish_sequence(ids[0])                                  # frees slot 1
    assert s.schedule_chunks([ids[3], ids[1]], [2, 1]).state_slots.tolist() == [1, 2]
    s.commit_chunks()
    for i in (1, 2, 3):
        s.finish_sequence(ids[i])
    assert s.is_finished() and s.get_stats()["free_blocks"] == 8
    again = s.add_sequence([1, 2, 3], sp)
    assert s.schedule_chunks([again], [3]).state_slots.tolist() == [0]


def test_models_without_state_carry_no_slots():
    from nano_vllm_rs_b200.engine import Config, SamplingParams, Scheduler
    s = Scheduler(Config("tiny", kvcache_block_size=16, num_kvcache_blocks=4, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64))
    a = s.add_sequence([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=1))
    assert s.schedule_chunks([a], [3]).state_slots is None


def test_regular_schedule_waits_for_a_slot_and_never_shares_pages():
    """Prefill-first scheduling of five equal prompts with three slots: three are admitted, the others wait until a running
    sequence finishes; equal prompts get pages of their own (a cached page cannot stand in for a recurrent state); a
    preempted sequence gives its slot back."""
    from nano_vllm_rs_b200.engine import SamplingParams
    s = stateful_sched(blocks=12, bs=4, seqs=3, batched=64)
    prompt = list(range(9))                                    # two full pages + one token: shareable if sharing were on
    ids = [s.add_sequence(prompt, SamplingParams(temperature=0.0, max_tokens=2 + i)) for i in range(5)]
    b = s.schedule()
    assert b.is_prefill and b.seq_ids.tolist() == ids[:3] and b.state_slots.tolist() == [0, 1, 2]
    assert b.input_ids.tolist() == prompt * 3 and s.get_stats()["cached_blocks"] == 0     # nothing skipped, nothing hashed
    assert s.get_stats()["used_blocks"] == 9 and len(set(b.slot_mapping.tolist())) == 27   # nine pages, every token its own slot
    s.postprocess([7, 7, 7])
    b = s.schedule()                                           # pages for a fourth prompt are free, a state slot is not
    assert not b.is_prefill and s.get_stats()["waiting"] == 2
    # run until everything is finished; slots in use never exceed three and are distinct in every batch
    steps = 0
    while not s.is_finished():
        s.postprocess([7] * len(b.seq_ids))
        if s.is_finished():
            break
        b = s.schedule()
        sl = b.state_slots.tolist()
        assert len(sl) == len(set(sl)) and all(0 <= x < 3 for x in sl)
        steps += 1
        assert steps < 100
    st = s.get_stats()
    assert st["finished"] == 5 and st["free_blocks"] == 12
