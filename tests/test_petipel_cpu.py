"""CPU: the host side of the Petipel model class — config parsing, registry, checkpoint container, the mixed-width
KV pool and its growth, the recurrent-state slot pool, the step's tile plan — and the oracle's own consistency."""
import json
import math

import pytest
import torch

import dgi_b200  # noqa: F401
from dgi_b200 import model_registry
from dgi_b200 import petipel_layer as P
from dgi_b200.paged_layer import RaggedBatchState
from dgi_b200.safetensors_io import read_safetensors, write_safetensors
from dgi_b200.worker.distributed.kv_cache import KVCachePool, RecurrentStatePool
from oracle import petipel_ref as R

CFG = {
    "architecture": "Petipel", "width": 24, "vocab": 29, "residual_mult": 0.5, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "hgrn2", "mixer": {"heads": 2, "dim": 6, "vdim": 10}, "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 6, "scale": 0.3, "bias_max": 30,
                                        "v_mix": True, "q_temp": {"coef": 0.4, "every": 4}},
         "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 3, "top": 2}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 12, "scale": 0.35, "bias_max": 9},
         "mlp": None},
    ],
}


def test_config_and_registry():
    cfg = P.PetipelConfig.from_dict(CFG)
    assert cfg.num_hidden_layers == 3 and cfg.hidden_size == 24 and cfg.vocab_size == 29
    assert cfg.kv_shape(0) is None and cfg.state_shape(0) == (2, 6, 10)
    assert cfg.kv_shape(1) == (2, 12, 6) and cfg.kv_shape(2) == (1, 8, 12) and cfg.state_shape(2) is None
    assert cfg.first_value_mix_layer() == 1
    assert model_registry.architecture_of(CFG).engine == "ragged"
    assert model_registry.architecture_of({"architectures": ["LlamaForCausalLM"]}).engine == "paged"
    with pytest.raises(KeyError):
        model_registry.architecture_of({"architecture": "nothing-known"})
    bad = json.loads(json.dumps(CFG))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(NotImplementedError):
        P.PetipelConfig.from_dict(bad)


def test_checkpoint_container_round_trip(tmp_path):
    cfg = P.PetipelConfig.from_dict(CFG)
    t = P.random_checkpoint(cfg, seed=1, bias_rows=10)
    assert t["l1.mix.rel"].shape == (10, 4) and t["l1.mix.vmix"].shape == () and t["l0.mix.f.b"].shape == (12,)
    assert t["l1.mlp.e2.down"].shape == (24, 8) and "l2.norm2" not in t and t["l2.mix.g"].shape == (2, 24)
    t["table"] = torch.arange(6, dtype=torch.int32).view(2, 3)
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, t)
    back = read_safetensors(path)
    assert sorted(back) == sorted(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and torch.equal(back[k], t[k]), k


def test_bucket_rule():
    assert [P.log_distance_bucket(n, 24, 100) for n in (0, 1, 11, 12, 13, 99, 100, 5000)] == \
        [0, 1, 11, 12, 12, 23, 23, 23]
    for rows, far in ((12, 40), (7, 20.5), (9, 64)):
        last = -1
        for n in range(0, 200):
            b = P.log_distance_bucket(n, rows, far)
            assert b == R.distance_bucket(n, rows, far) and last <= b <= rows - 1
            last = b
        assert P.log_distance_bucket(int(math.ceil(far)), rows, far) == rows - 1
        lut = P.distance_bias_table(torch.arange(rows, dtype=torch.float32)[:, None], far)
        assert lut.shape[0] == 1 and lut[0, -1] == rows - 1 and lut[0, 0] == 0


def test_mixed_width_pool_grows_and_reuses_pages():
    pool = KVCachePool(2, 0, 0, 16, 6, "cpu", torch.float32, layer_shapes=[(2, 12, 6), (1, 8, 12)])
    assert pool.layer(0).key_pool.shape == (6, 2, 16, 12) and pool.layer(0).value_pool.shape == (6, 2, 16, 6)
    assert pool.layer(1).key_pool.shape == (6, 1, 16, 8) and pool.layer(1).value_pool.shape == (6, 1, 16, 12)
    a = pool.allocate_sequence(0)
    assert a == [[], []]
    pool.extend_sequence(a, 17)
    pool.extend_sequence(a, 20)      # still two pages
    b = pool.allocate_sequence(33)
    assert [len(x) for x in a] == [2, 2] and [len(x) for x in b] == [3, 3]
    assert KVCachePool.block_table(a[0]) == KVCachePool.block_table(a[1])
    for li in range(2):              # live sequences pin their pages (unpinned pages are an evictable cache)
        pool.layer(li).pin(blk.block_id for blk in a[li] + b[li])
    with pytest.raises(RuntimeError):
        pool.extend_sequence(a, 49)  # needs two more pages, one is free: nothing is taken
    assert [len(x) for x in a] == [2, 2] and len(pool.layer(0)._free_blocks) == 1 and len(pool.layer(1)._free_blocks) == 1
    freed = KVCachePool.block_table(b[0])
    pool.free_sequence(b)
    pool.extend_sequence(a, 49)
    assert set(KVCachePool.block_table(a[0])[2:]) <= set(freed) | {0, 1, 2, 3, 4, 5}
    assert len(set(KVCachePool.block_table(a[0]))) == 4


def test_state_pool_slots():
    sp = RecurrentStatePool([(2, 6, 10), (1, 3, 4)], 3, "cpu")
    assert sp.layer(0).shape == (3, 2, 6, 10) and sp.layer(1).dtype == torch.float32
    s0, s1, s2 = sp.allocate(), sp.allocate(), sp.allocate()
    assert sorted((s0, s1, s2)) == [0, 1, 2] and sp.free_slots == 0
    with pytest.raises(RuntimeError):
        sp.allocate()
    sp.layer(0)[s1].fill_(3.0)
    sp.free(s1)
    with pytest.raises(ValueError):
        sp.free(s1)
    assert sp.allocate() == s1          # last freed, first reused — with its old content until reset
    assert float(sp.layer(0)[s1].max()) == 3.0
    sp.reset(s1)
    assert float(sp.layer(0)[s1].abs().max()) == 0.0


def test_tile_plan_keeps_sequences_apart():
    st = RaggedBatchState(tok_pos=torch.zeros(1, dtype=torch.int32), slot_mapping=torch.zeros(1, dtype=torch.int64),
                          block_tables=torch.zeros((3, 1), dtype=torch.int32),
                          scan_seqs=torch.zeros((3, 4), dtype=torch.int32),
                          spans=[(0, 19, 0, 100), (19, 1, 1, 7), (20, 8, 2, 0)])
    tiles, most = st.tiles_for(4, 1)            # 8 tokens x 4 heads of a group = 32 rows per CTA
    rows = tiles.tolist()
    assert most == 8 and sorted(rows) == sorted([[0, 8, 0], [8, 8, 0], [16, 3, 0], [19, 1, 1], [20, 8, 2]])
    assert rows[0] == [16, 3, 0]                # longest context first
    tiles2, most2 = st.tiles_for(8, 8)          # one head per group: 32 tokens per CTA
    assert most2 == 19 and sorted(tiles2.tolist()) == [[0, 19, 0], [19, 1, 1], [20, 8, 2]]


def test_oracle_recurrence_carries_its_state():
    cfg = P.PetipelConfig.from_dict(CFG)
    t = {k[len("l0.mix."):]: v.float() for k, v in P.random_checkpoint(cfg, seed=2).items() if k.startswith("l0.mix.")}
    h = torch.randn(11, 24, generator=torch.Generator().manual_seed(0))
    whole, S = R.hgrn2_mixer(h, t, CFG["layers"][0]["mixer"], 1e-5)
    a, Sa = R.hgrn2_mixer(h[:4], t, CFG["layers"][0]["mixer"], 1e-5)
    b, Sb = R.hgrn2_mixer(h[4:], t, CFG["layers"][0]["mixer"], 1e-5, state=Sa)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-6) and torch.allclose(Sb, S, atol=1e-6)
    logits = R.forward(CFG, P.random_checkpoint(cfg, seed=2, bias_rows=10), [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, 29) and torch.isfinite(logits).all()
