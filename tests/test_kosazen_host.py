"""CPU tests around the Kosazen integration: the oracle's own mechanisms (properties that hold by construction), the model
registry's configuration reader, and the scheduler's explicit portion stepping (block accounting, reuse, refusals)."""
import json

import numpy as np
import pytest

from oracle import kosazen as K


# ------------------------------------------------------------------------------------------------ oracle properties


def test_rotation_depends_on_distance_only():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal(8), rng.standard_normal(8)
    d = lambda pq, pk: K.rotate_pairs(q, pq, 6, 300.0) @ K.rotate_pairs(k, pk, 6, 300.0)
    assert abs(d(17, 5) - d(112, 100)) < 1e-9 and abs(d(17, 5) - d(17, 6)) > 1e-6
    assert np.allclose(K.rotate_pairs(q, 9, 6, 300.0)[6:], q[6:])           # beyond `dims` nothing moves
    assert np.allclose(K.rotate_pairs(q, 0, 6, 300.0), q)


def test_router_weights_and_identity_experts():
    rng = np.random.default_rng(1)
    W, E, I = 6, 2, 2
    w = {"router": rng.standard_normal((E + I, W)), "correction": np.zeros(E + I)}
    h = rng.standard_normal(W)
    r = {"experts": E, "identity": I, "top": 2, "scale": 1.7}
    idx, wt, _ = K.route(h, w, "", r)
    assert abs(wt.sum() - 1.7) < 1e-12
    w["correction"] = np.array([-9.0, -9.0, 0.0, 0.0])                      # only identity experts can be chosen
    f = {"router": r, "expert": {"ff": 3, "limit": 1.0}}
    np.testing.assert_allclose(K.moe(h, w, "", f), 1.7 * h)
    # the bias steers the choice, the weights come from the unbiased softmax
    w["correction"] = np.array([0.0, 5.0, 0.0, 0.0])
    idx2, wt2, _ = K.route(h, w, "", dict(r, top=1))
    assert idx2[0] == 1 and abs(wt2[0] - 1.7) < 1e-12


def test_gated_expert_clamps():
    wg, wu, wd = np.eye(2), np.eye(2), np.eye(2)
    out = K.glu_expert(np.array([10.0, -10.0]), wg, wu, wd, 2.0)
    g = np.array([2.0, -10.0])                                               # the gate is capped from above only
    np.testing.assert_allclose(out, g / (1 + np.exp(-1.702 * g)) * (np.array([2.0, -2.0]) + 1))


def test_loop_order_and_cache_per_run():
    cfg = K.random_config(np.random.default_rng(2), n_layers=4, loop=(1, 3, 3))
    assert K.layer_runs(cfg) == [0, 1, 2, 1, 2, 1, 2, 3]
    cfg.pop("loop")
    assert K.layer_runs(cfg) == [0, 1, 2, 3]
    assert len(K.Sequence(K.random_config(np.random.default_rng(2), n_layers=4, loop=(1, 3, 3))).cache) == 8


def test_oracle_state_is_per_sequence():
    rng = np.random.default_rng(3)
    cfg = K.random_config(rng, n_layers=2, vocab=20, width=12)
    w = K.random_weights(cfg, rng)
    a, b = [3, 7, 1, 9], [5, 5, 2]
    sa, sb = K.Sequence(cfg), K.Sequence(cfg)
    inter = []
    for i in range(4):
        inter.append(K.step_token(cfg, w, sa, a[i]))
        if i < 3:
            K.step_token(cfg, w, sb, b[i])
    np.testing.assert_allclose(np.stack(inter), K.logits_of(cfg, w, a), rtol=1e-12)


# ------------------------------------------------------------------------------------------------ registry / configuration


def test_model_registry_reads_config_json():
    from nano_vllm_rs_b200.engine import Config, lib
    assert b"Kosazen" in lib().nvllm_registered_architectures()
    cfg = K.random_config(np.random.default_rng(4), n_layers=3, loop=(1, 2, 4), vocab=77, width=24)
    c = Config(model_config=json.dumps(cfg))
    assert (c.arch, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Kosazen", 77, 24, 6)   # layer RUNS: 1 + 4 + 1
    c2 = Config(model_config=cfg, dtype="float32", kvcache_block_size=48, max_num_seqs=3)
    assert c2.kvcache_block_size == 48 and c2.dtype == "float32"


@pytest.mark.parametrize("breakage,needle", [
    (lambda c: c.update(architecture="Nonesuch"), "Nonesuch"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="windowed"), "windowed"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=99), "router"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
])
def test_bad_model_configs_are_refused_with_a_reason(breakage, needle):
    from nano_vllm_rs_b200 import _ffi
    from nano_vllm_rs_b200.engine import Config
    cfg = K.random_config(np.random.default_rng(5), n_layers=2)
    breakage(cfg)
    with pytest.raises(_ffi.NvllmError) as e:
        Config(model_config=json.dumps(cfg))
    assert needle in str(e.value)
    with pytest.raises(_ffi.NvllmError):
        Config(model_config="{not json")
    with pytest.raises(ValueError):
        Config("qwen3-0.6b", dtype="float32")


# ------------------------------------------------------------------------------------------------ explicit stepping


def small_sched(blocks=6, bs=16, seqs=3):
    from nano_vllm_rs_b200.engine import Config, Scheduler
    cfg = Config("tiny", kvcache_block_size=bs, num_kvcache_blocks=blocks, max_num_seqs=seqs, max_num_batched_tokens=64,
                 max_model_len=blocks * bs)
    return Scheduler(cfg)


def test_portions_take_pages_as_they_grow_and_give_them_back():
    from nano_vllm_rs_b200.engine import SamplingParams
    s = small_sched()
    sp = SamplingParams(temperature=0.0, max_tokens=1)
    a = s.add_sequence(list(range(10)), sp)
    b = s.schedule_chunks([a], [10])
    assert b.is_prefill and b.block_tables is not None and b.positions.tolist() == list(range(10))
    assert b.slot_mapping.tolist() == list(range(10)) and b.cu_seqlens_q.tolist() == [0, 10] and b.cu_seqlens_k.tolist() == [0, 10]
    s.commit_chunks()
    assert s.get_stats()["used_blocks"] == 1
    s.extend_sequence(a, list(range(100, 130)))                      # 40 tokens now; run 7 of them beside a new request
    c = s.add_sequence([1, 2, 3], sp)
    b = s.schedule_chunks([c, a], [2, 7])
    assert b.positions.tolist() == [0, 1] + list(range(10, 17)) and b.input_ids.tolist() == [1, 2] + list(range(100, 107))
    assert b.cu_seqlens_q.tolist() == [0, 2, 9] and b.cu_seqlens_k.tolist() == [0, 2, 19]
    # request a crossed into its second page (taken after c's first): slots of positions 16.. lie in block 2
    assert b.slot_mapping.tolist() == [16, 17] + list(range(10, 16)) + [32]
    assert b.block_tables.tolist() == [[1, -1], [0, 2]]
    s.commit_chunks()
    b = s.schedule_chunks([a, c], [23, 1])
    assert b.positions.tolist() == list(range(17, 40)) + [2] and b.block_tables.tolist() == [[0, 2, 3], [1, -1, -1]]
    s.commit_chunks()
    assert s.get_stats()["used_blocks"] == 4 and s.get_stats()["running"] == 2
    s.finish_sequence(a)
    s.release_sequence(a)
    assert s.get_stats()["used_blocks"] == 1 and s.free_list() == [4, 5, 3, 2, 0]
    d = s.add_sequence(list(range(40)), sp)                          # takes freed pages again, in free-list order
    b = s.schedule_chunks([d], [40])
    assert b.block_tables.tolist() == [[4, 5, 3]]
    s.commit_chunks()
    s.finish_sequence(d); s.finish_sequence(c)
    assert s.get_stats()["free_blocks"] == 6 and s.is_finished()


def test_portion_steps_are_refused_without_side_effects():
    from nano_vllm_rs_b200 import _ffi
    from nano_vllm_rs_b200.engine import SamplingParams
    s = small_sched(blocks=2)
    sp = SamplingParams(temperature=0.0, max_tokens=1)
    a, b = s.add_sequence(list(range(20)), sp), s.add_sequence(list(range(20)), sp)
    for ids, counts in (([a], [21]), ([a], [0]), ([a, a], [1, 1]), ([a, 99], [1, 1]), ([a, b], [20, 20])):   # last: 4 pages of 2
        with pytest.raises(_ffi.NvllmError):
            s.schedule_chunks(ids, counts)
        assert s.get_stats()["used_blocks"] == 0 and s.get_stats()["waiting"] == 2
    s.schedule_chunks([a, b], [16, 16])
    s.commit_chunks()
    with pytest.raises(_ffi.NvllmError):
        s.schedule_chunks([a], [4])                                   # no page left for position 16
    s.finish_sequence(b)
    assert s.schedule_chunks([a], [4]).slot_mapping.tolist() == [16, 17, 18, 19]   # b's page, used again
    with pytest.raises(_ffi.NvllmError):
        s.extend_sequence(b, [1])                                     # finished
    with pytest.raises(_ffi.NvllmError):
        s.extend_sequence(a, list(range(100)))                        # beyond max_model_len


def test_loader_accepts_scalar_tensors(tmp_path):
    from nano_vllm_rs_b200.loader import ModelLoader, write_safetensors

    class Sink:
        def __init__(self): self.got = {}
        def load_weight(self, name, bits): self.got[name] = bits

    write_safetensors(str(tmp_path / "m.safetensors"), {"x.alpha": K.to_bf16_bits(np.asarray(1.5)), "v": K.to_bf16_bits(np.ones(3))})
    sink = Sink()
    assert ModelLoader(sink).load_safetensors(str(tmp_path / "m.safetensors")) == 2
    assert sink.got["x.alpha"].shape == (1,) and sink.got["x.alpha"][0] == 0x3FC0 and sink.got["v"].shape == (3,)
