"""CPU: configuration, registry, pools and checkpoint layout of the Sanesun model class, and sanity of its oracle."""
import math

import pytest
import torch

import dgi_b200  # noqa: F401
from dgi_b200 import model_registry
from dgi_b200 import sanesun_layer as S
from dgi_b200.worker.distributed.kv_cache import KVCachePool, RecurrentStatePool
from oracle import sanesun_ref as R

CFG = {
    "architecture": "Sanesun", "width": 24, "vocab": 19, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "conv": 3}, "mlp": {"kind": "dense", "ff": 30}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 4, "vdim": 6, "kv_rank": 10, "q_rank": 12, "scale": 0.5}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.35,
                                       "mask": {"size": 7, "keep_first": 2}, "rot": {"base": 100.0, "dims": 4}},
         "mlp": {"kind": "dense", "ff": 12}},
    ],
}


def test_config_names_pools_and_states():
    cfg = S.SanesunConfig.from_dict(CFG)
    assert cfg.num_hidden_layers == 3 and cfg.hidden_size == 24 and cfg.vocab_size == 19 and cfg.embed_scale == 2.0
    assert cfg.kv_shape(0) is None and cfg.state_shape(0) == [(4, 6, 10), (2, 2 * 2 * 6 + 4 * 10)]
    assert cfg.kv_shape(1) == (1, 10, 0) and cfg.state_shape(1) is None      # one latent row per token, no value pool
    assert cfg.kv_shape(2) == (2, 8, 6) and cfg.state_shape(2) is None
    bad = dict(CFG, layers=[dict(CFG["layers"][0], type="conv_only")])
    with pytest.raises(NotImplementedError):
        S.SanesunConfig.from_dict(bad)
    assert model_registry.architecture_of(CFG).name == "Sanesun"
    assert "Sanesun" in model_registry.known_architectures()


def test_state_pool_groups_and_key_only_pages():
    pool = RecurrentStatePool([[(4, 6, 10), (2, 64)], (3, 5, 5)], slots=3, device="cpu")
    state, tail = pool.layer(0)
    assert tuple(state.shape) == (3, 4, 6, 10) and tuple(tail.shape) == (3, 2, 64) and tuple(pool.layer(1).shape) == (3, 3, 5, 5)
    a, b = pool.allocate(), pool.allocate()
    tail[b].fill_(1.0)
    pool.reset(b)
    assert tail[b].abs().sum() == 0 and (a, b) == (0, 1)
    pool.free(a)
    assert pool.allocate() == a and pool.get_total_memory_gb() > 0
    kv = KVCachePool(num_layers=2, num_heads=0, head_dim=0, block_size=16, max_blocks_per_layer=4, device="cpu",
                     dtype=torch.float32, layer_shapes=[(1, 10, 0), (2, 8, 6)])
    assert tuple(kv.layer(0).key_pool.shape) == (4, 1, 16, 10) and kv.layer(0).value_pool.numel() == 0
    assert tuple(kv.layer(1).value_pool.shape) == (4, 2, 16, 6)


def test_random_checkpoint_has_the_checkpoint_names():
    cfg = S.SanesunConfig.from_dict(CFG)
    t = S.random_checkpoint(cfg, seed=1)
    assert tuple(t["l0.mix.q.conv"].shape) == (12, 3) and tuple(t["l0.mix.v"].shape) == (40, 24)
    assert tuple(t["l0.mix.a2"].shape) == (24, t["l0.mix.a1"].shape[0]) and tuple(t["l0.mix.dt_bias"].shape) == (24,)
    assert tuple(t["l1.mix.uk"].shape) == (12, 10) and tuple(t["l1.mix.uv"].shape) == (18, 10) and "l1.mlp.up" not in t
    assert tuple(t["l2.mix.talk"].shape) == (4, 4) and tuple(t["l2.mix.sink"].shape) == (4,) and "l2.mix.q.b" in t
    logits = R.forward(CFG, t, [1, 5, 7, 2, 2, 18, 0, 3, 9, 11])
    assert logits.shape == (10, 19) and torch.isfinite(logits).all()


def test_oracle_properties():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.arange(5)
    back = R.turn(R.turn(x, pos, 8, 50.0), pos, 8, 50.0, back=True)
    assert (back - x).abs().max() < 1e-12
    part = R.turn(x, pos, 4, 50.0)
    assert (part[..., 4:] == x[..., 4:]).all() and (part[0] == x[0]).all()          # position 0 turns nothing
    # with decay 1 and write strength 1 the delta rule stores v exactly under a unit key and returns it for q = k
    n, dk, dv = 3, 4, 2
    k = torch.eye(dk, dtype=torch.float64)[:n].view(n, 1, dk)
    v = torch.randn(n, 1, dv, generator=g, dtype=torch.float64)
    o = R.delta_rule(k, k, v, torch.ones(n, 1, dtype=torch.float64), torch.ones(n, 1, dk, dtype=torch.float64))
    assert (o - v).abs().max() < 1e-12
    # causal_conv_silu: a one-tap filter of ones is SiLU
    z = torch.randn(6, 3, generator=g, dtype=torch.float64)
    assert (R.causal_conv_silu(z, torch.ones(3, 1, dtype=torch.float64)) - z * torch.sigmoid(z)).abs().max() < 1e-12
    # a window as long as the sequence with nothing kept is plain causal attention
    q, kk, vv = (torch.randn(7, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    assert (R.windowed_attention(q, kk, vv, 0.5, 7, 0) - R.windowed_attention(q, kk, vv, 0.5)).abs().max() < 1e-12
    assert math.isclose(float(R.xielu(torch.tensor(0.0, dtype=torch.float64), torch.tensor(0.3), torch.tensor(0.2))), 0.0)
