"""The Zanelorn configuration reader, its lowering to a plan and the plain implementation's own
mechanisms (no GPU)."""
import copy
import math

import pytest
import torch

import plain_zanelorn as P
from zanelorn_cases import ZAN_A, ZAN_B, ZAN_C, ZAN_D
from minfer_b200.config.base import ConfigError
from minfer_b200.model import Model
from minfer_b200.registry import read_config


def test_reads_every_size_and_constant():
    cfg = read_config(ZAN_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (97, 64, 1e-6)
    assert (cfg.residual_mult, cfg.embedding_scale, cfg.side_dim) == (0.6, 3.0, 8)
    plan = cfg.plan()
    assert plan.embedding_scale == 3.0
    assert [l.mixer.kind for l in plan.layers] == ["parallel", "retention", "retention", "parallel"]
    assert all(l.block.kind == "output_norm" and l.block.params["mult"] == 0.6 for l in plan.layers)
    assert [l.block.params["side"]["offset"] for l in plan.layers] == [0, 8, 16, 24]
    assert plan.layers[0].block.params["side"]["table_width"] == 32
    par = plan.layers[0].mixer.params
    att, scan = par["left"].params, par["right"].params
    assert (par["left_scale"], par["right_scale"]) == (0.7, 1.2)
    assert (att["n_heads"], att["n_kv_heads"], att["head_dim"], att["value_dim"]) == (4, 2, 16, 24)
    assert (att["window"], att["keep_first"], att["scale"]) == (20, 3, 0.3)
    assert att["norm_scope"] == "head" and att["gate"] and att["bias"]
    rot = att["position"].params
    assert (rot["rotary_dim"], rot["theta"], rot["frequency_scale"], rot["style"]) == (8, 50000.0, 0.5, "neox")
    assert (scan["inner"], scan["n_state"], scan["dt_rank"], scan["conv"]) == (48, 8, 5, 3)
    ret = plan.layers[1].mixer.params
    assert (ret["n_heads"], ret["head_dim"], ret["value_dim"]) == (3, 12, 20)
    assert ret["decay"] == [0.9, 0.97, 0.995] and ret["position"].params["rotary_dim"] == 12
    moe = plan.layers[1].feed_forward.params
    assert (moe["n_experts"], moe["identity"], moe["top"], moe["intermediate_size"]) == (5, 1, 2, 24)
    assert moe["limit"] == 1.2 and moe["shared"]["ff"] == 40 and moe["shared"]["limit"] == 0.9
    assert moe["scoring"] == "softmax_all" and moe["activation"] == "clamped_swish"
    assert plan.layers[2].feed_forward is None and plan.layers[2].feed_forward_norm is None
    assert plan.layers[0].feed_forward.kind == "dense_mlp"
    assert plan.layers[0].feed_forward.params["activation"] == "gelu"
    assert read_config(cfg.to_dict()) == cfg


def test_defaults_and_absent_keys():
    cfg = read_config(ZAN_B)
    assert (cfg.residual_mult, cfg.embedding_scale, cfg.side_dim) == (1.0, 1.0, 0)
    plan = cfg.plan()
    assert all(l.block.params["side"] is None for l in plan.layers)
    assert plan.layers[0].mixer.params["position"] is None             # retention without a rotation
    att = plan.layers[1].mixer.params["left"].params
    assert (att["window"], att["keep_first"]) == (0, 0)                # no mask at all
    assert att["position"].params["frequency_scale"] == pytest.approx(1 / 3.0)
    assert plan.layers[2].mixer.params["left"].params["position"].params["frequency_scale"] == 1.0
    moe = plan.layers[0].feed_forward.params
    assert moe["identity"] == 0 and moe["shared"] is None and moe["top"] == 1


def test_tensor_names_and_shapes():
    cfg = read_config(ZAN_A)
    specs = {s.name: tuple(s.shape) for s in Model(cfg.plan(), "float32", cfg).tensor_specs()}
    assert specs["embed"] == (97, 64) and specs["head"] == (97, 64) and specs["final.norm"] == (64,)
    assert specs["side.embed"] == (97, 32)                             # one table for all layers
    for n, shape in {"l0.mix.left.q": (64, 64), "l0.mix.left.q.b": (64,), "l0.mix.left.k": (32, 64),
                     "l0.mix.left.v": (48, 64), "l0.mix.left.v.b": (48,), "l0.mix.left.q.norm": (16,),
                     "l0.mix.left.k.norm": (16,), "l0.mix.left.g": (96, 64), "l0.mix.left.o": (64, 96),
                     "l0.mix.right.in": (96, 64), "l0.mix.right.conv": (48, 3), "l0.mix.right.conv.b": (48,),
                     "l0.mix.right.x": (21, 48), "l0.mix.right.dt": (48, 5), "l0.mix.right.dt.b": (48,),
                     "l0.mix.right.A_log": (48, 8), "l0.mix.right.D": (48,), "l0.mix.right.o": (64, 48),
                     "l0.mlp.up": (48, 64), "l0.mlp.down": (64, 48), "l0.norm1": (64,), "l0.norm2": (64,),
                     "l0.side.gate": (8, 64), "l0.side.proj": (64, 8), "l0.side.norm": (64,),
                     "l1.mix.q": (36, 64), "l1.mix.k": (36, 64), "l1.mix.v": (60, 64), "l1.mix.g": (60, 64),
                     "l1.mix.o": (64, 60), "l1.mlp.router": (6, 64), "l1.mlp.correction": (6,),
                     "l1.mlp.e4.gate": (24, 64), "l1.mlp.e0.down": (64, 24), "l1.mlp.shared.gate": (40, 64),
                     "l1.mlp.shared.down": (64, 40), "l1.mlp.shared.sg": (1, 64),
                     "l3.mlp.router": (6, 64)}.items():
        assert specs[n] == shape, n
    assert "l1.mlp.e5.gate" not in specs and "l2.norm2" not in specs and "l2.mlp.up" not in specs
    assert "l3.mlp.shared.gate" not in specs


@pytest.mark.parametrize("change,where", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_refusals(change, where):
    cfg = copy.deepcopy(ZAN_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        read_config(cfg)
    assert where in str(e.value)


def test_every_case_reads_and_registers():
    for c in (ZAN_A, ZAN_B, ZAN_C, ZAN_D):
        cfg = read_config(c)
        model = Model(cfg.plan(), "bfloat16", cfg)
        assert len(model.blocks) == len(c["layers"])


# ---- the plain implementation's own mechanisms, against closed forms ---------------------------
def test_plain_visibility():
    see = P.visible(12, 4, 2)
    assert see[11].nonzero().flatten().tolist() == [0, 1, 8, 9, 10, 11]
    assert see[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert see[5].nonzero().flatten().tolist() == [0, 1, 2, 3, 4, 5]
    assert P.visible(5, 100, 0).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()


def test_plain_retention_is_a_decayed_sum():
    """With one head and no rotation, o_t = sum_{s <= t} a^(t-s) (q_t . k_s) v_s D^(-1/2)."""
    torch.manual_seed(0)
    T, W, D, Dv, a = 9, 6, 4, 5, 0.8
    w = {"q": torch.randn(D, W).double(), "k": torch.randn(D, W).double(), "v": torch.randn(Dv, W).double(),
         "g": torch.zeros(Dv, W).double(), "o": torch.eye(Dv).double()}
    x = torch.randn(T, W).double()
    q, k, v = x @ w["q"].T, x @ w["k"].T, x @ w["v"].T
    want = torch.zeros(T, Dv).double()
    for t in range(T):
        for s in range(t + 1):
            want[t] += a ** (t - s) * float(q[t] @ k[s]) * D ** -0.5 * v[s]
    # a zero gate projection gives silu(0) = 0; use a gate of ones through a bias-free trick instead
    w["g"] = torch.zeros(Dv, W).double()
    x1 = torch.cat([x, torch.ones(T, 1).double()], dim=1)
    w1 = {n: torch.cat([m, torch.zeros(m.shape[0], 1).double()], dim=1) for n, m in w.items() if n != "o"}
    w1["g"][:, -1] = 20.0                                              # silu(20) = 20 to 1e-8
    w1["o"] = w["o"]
    got = P.retention(x1, w1, "", {"heads": 1, "dim": D, "vdim": Dv, "decay": [a]}, 0.0)
    assert torch.allclose(got, P.rms_unit(want, 0.0) * 20.0, atol=1e-6)


def test_plain_rotation_is_relative():
    """(rotated q_i) . (rotated k_j) depends on i - j only."""
    torch.manual_seed(1)
    q, k = torch.randn(1, 1, 8).double(), torch.randn(1, 1, 8).double()
    qs, ks = q.repeat(20, 1, 1), k.repeat(20, 1, 1)
    rq, rk = P.rotate_half(qs, 6, 100.0, 2.0), P.rotate_half(ks, 6, 100.0, 2.0)
    a = float(rq[7, 0] @ rk[3, 0])
    b = float(rq[19, 0] @ rk[15, 0])
    assert abs(a - b) < 1e-12
    assert torch.equal(rq[..., 6:], qs[..., 6:])                        # the rest passes unchanged
    ang = 5 * 100.0 ** (-2.0 / 6) / 2.0                                 # pair (1, 4) at position 5
    assert abs(float(rq[5, 0, 1]) - (float(q[0, 0, 1]) * math.cos(ang) - float(q[0, 0, 4]) * math.sin(ang))) < 1e-12


def test_plain_router():
    w = {"router": torch.eye(4).double() * 3, "correction": torch.tensor([0.0, 0.0, 0.9, 0.0]).double()}
    x = torch.tensor([[1.0, 0.5, 0.0, 0.2]]).double()
    chosen, weight, _ = P.route(x, w, "", 2)
    s = torch.softmax(x @ w["router"].T, dim=-1)
    assert chosen.tolist() == [[2, 0]]                                  # the correction lifts expert 2
    assert torch.allclose(weight, s[:, [2, 0]])                         # weights: the plain scores
