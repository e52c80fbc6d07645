"""CPU tests of the host-side mirror: config defaults, gate/activation mapping, stats."""
import numpy as np
import pytest


def test_config_defaults_match_reference(lib_built):
    import mixtureofexperts_b200 as m

    c = m.create_moe_config()
    # src/core/moe_layer.jl:4-29
    assert (c.num_experts, c.expert_type, c.input_dim, c.hidden_dim, c.output_dim) == (8, "standard", 768, 3072, 768)
    assert c.activation is m.gelu and isinstance(c.gate_type, m.TopKGating) and c.gate_type.k == 2
    assert c.z_loss_weight == pytest.approx(0.001) and c.capacity_factor == 1.25 and not c.drop_tokens
    assert isinstance(c.balance_loss, m.SwitchTransformerLoss) and c.balance_loss.alpha == pytest.approx(0.01)
    assert c.num_shared_experts == 0 and c.use_fp32_router


def test_gate_mapping(lib_built):
    import mixtureofexperts_b200 as m
    from mixtureofexperts_b200 import _lib
    from mixtureofexperts_b200.gating import gate_kind_of

    assert gate_kind_of(m.TopKGating(3)) == (_lib.GATE_TOPK, 3, 0)
    assert gate_kind_of(m.SwitchGating()) == (_lib.GATE_SWITCH, 1, 0)
    assert gate_kind_of(m.SharedExpertGating(2, m.TopKGating(6), 66)) == (_lib.GATE_SHARED_TOPK, 6, 2)
    with pytest.raises(m.MoEError):
        gate_kind_of(object())


def test_activation_mapping_by_identity_and_by_probe(lib_built):
    import mixtureofexperts_b200 as m
    from mixtureofexperts_b200 import _lib
    from mixtureofexperts_b200.layer import activation_enum

    assert activation_enum(m.silu) == _lib.ACT_SILU
    assert activation_enum(m.gelu) == _lib.ACT_GELU_TANH
    assert activation_enum("relu") == _lib.ACT_RELU
    # convert_to_moe passes an anonymous x -> x*sigmoid(x) (src/llama2/conversion.jl:212)
    assert activation_enum(lambda x: x * (1.0 / (1.0 + np.exp(-x)))) == _lib.ACT_SILU
    assert activation_enum(lambda x: max(x, 0.0)) == _lib.ACT_RELU
    with pytest.raises(m.MoEError):
        activation_enum(lambda x: x * x)


def test_load_balance_score(lib_built):
    import mixtureofexperts_b200 as m

    assert m.load_balance_score([5, 5, 5, 5]) == pytest.approx(1.0)
    assert m.load_balance_score([0, 0, 0, 0]) == 1.0
    assert m.load_balance_score([10, 0]) == pytest.approx(0.0)


def test_aux_free_bias_update(lib_built):
    import mixtureofexperts_b200 as m

    loss = m.AuxiliaryFreeLoss(4)
    loss.update_bias([10, 0, 0, 0])
    # the overloaded expert's bias goes down, the mean stays 0 (auxiliary_free.jl:60-70)
    assert loss.bias[0] < 0 and abs(float(loss.bias.sum())) < 1e-6 and (loss.bias[1:] > 0).all()


def test_aux_free_host_update_equals_the_oracle(lib_built):
    import mixtureofexperts_b200 as m
    from oracle import moe_oracle as orc

    rng = np.random.default_rng(0)
    loss = m.AuxiliaryFreeLoss(6, learning_rate=0.5, momentum=0.7, update_freq=2)
    st = orc.AuxFreeState(bias=np.zeros(6, dtype=np.float32), bias_momentum=np.zeros(6, dtype=np.float32),
                          learning_rate=0.5, momentum=0.7, update_freq=2)
    for _ in range(7):
        idx = rng.integers(0, 7, size=(40, 2))                  # 0 = dropped slot
        orc.aux_free_update_bias(st, idx)
        loss.update_bias(np.bincount(idx.reshape(-1), minlength=7)[1:])
        assert np.array_equal(loss.bias, st.bias) and np.array_equal(loss.bias_momentum, st.bias_momentum)
    assert loss.update_counter == 7


def test_gated_expert_init_scale(lib_built):
    import mixtureofexperts_b200 as m

    e = m.GatedExpert(256, 512, 256, m.silu, rng=0)
    assert e.w1.shape == (512, 256) and e.w2.shape == (256, 512) and e.w3.shape == (512, 256)
    # all three use sigma = sqrt(2/input_dim) (src/experts/gated.jl:16-24)
    for w in (e.w1, e.w2, e.w3):
        assert abs(float(w.std()) - (2.0 / 256) ** 0.5) < 0.01


def test_standard_expert_init_scale_and_bias(lib_built):
    import mixtureofexperts_b200 as m

    e = m.StandardExpert(256, 512, 128, m.gelu, rng=0)
    assert e.w1.shape == (512, 256) and e.w2.shape == (128, 512)
    # sigma1 = sqrt(2/input_dim), sigma2 = sqrt(2/hidden_dim), zero biases (src/experts/standard.jl:21-32)
    assert abs(float(e.w1.std()) - (2.0 / 256) ** 0.5) < 0.01
    assert abs(float(e.w2.std()) - (2.0 / 512) ** 0.5) < 0.01
    assert e.b1.shape == (512,) and e.b2.shape == (128,) and not e.b1.any() and not e.b2.any()
    nb = m.StandardExpert(8, 8, 8, m.gelu, bias=False)
    assert nb.b1 is None and nb.b2 is None
    with pytest.raises(ValueError):
        m.StandardExpert(8, 8, 8, m.gelu, dropout=0.1)


def test_router_noise_network_init(lib_built):
    import mixtureofexperts_b200 as m

    r = m.Router(64, 8, m.TopKGating(2), noise_scale=0.1, use_noise_network=True, rng=0)
    lim = (6.0 / (64 + 8)) ** 0.5                       # Flux Dense default init, like Router.weight
    assert r.noise_weight.shape == (8, 64) and np.abs(r.noise_weight).max() <= lim
    assert not np.array_equal(r.noise_weight, r.weight)
    assert m.Router(64, 8, m.TopKGating(2)).noise_weight is None
