"""The sample-input factories and shape contracts (CPU: no kernel is called)."""
import torch

from retention_integration_b200 import create_inputs as ci
from retention_integration_b200 import layout


def _check(props, tensors):
    for name, spec in props.items():
        if spec is None:
            assert tensors.get(name) is None, name
            continue
        shape, dtype, device = spec
        x = tensors[name]
        assert tuple(x.shape) == tuple(shape) and x.dtype == dtype and x.device.type == torch.device(device).type, name


def test_training_inputs_match_their_contract_and_are_deterministic():
    kw = dict(b=2, t=96, h=3, d=32, qhead_ratio=2, dtype=torch.bfloat16, device="cpu", gating=True, chunk_size=32)
    a, b = ci.create_inputs(**kw), ci.create_inputs(**kw)
    _check(ci.input_properties(**kw), a)
    for k in ("Q", "K", "V", "log_G"):
        assert torch.equal(a[k], b[k])
    assert a["log_G"].max() <= 0 and a["scale"] == 1.0 and a["chunk_size"] == 32
    assert ci.output_properties(**kw)["Y"][0] == (2, 96, 6, 32)
    g = ci.create_inputs(requires_grad=True, **kw)
    assert all(g[k].requires_grad and g[k].is_leaf for k in ("Q", "K", "V", "log_G"))


def test_inference_inputs_match_their_contract():
    kw = dict(b=1, tq=1, tk=64, h=2, d=64, qhead_ratio=12, dtype=torch.bfloat16, device="cpu", gating=True,
              initial_state=True, switch_over_seq_len=128)
    x = ci.create_inference_inputs(**kw)
    _check(ci.inference_input_properties(**kw), x)
    assert x["initial_state"].shape == (1, 2, layout.exact_dim(64), 64) and (x["sum_of_keys"] >= 0).all()
    out = ci.inference_output_properties(**kw)
    assert out["state"][0] == (1, 2, 2080, 64) and out["sum_of_keys"][1] == torch.float32
    no_state = ci.inference_output_properties(**{**kw, "initial_state": False})
    assert no_state["state"] is None  # 64 cached tokens < switch-over 128 and nothing carried in
    assert ci.inference_output_properties(**{**kw, "initial_state": False, "tk": 128})["state"] is not None
    y = ci.create_inference_inputs(**{**kw, "tk": 0})
    assert y["K"] is None and y["log_G"] is None


def test_grids_cover_the_reference_tables():
    assert len(ci.grid_cases(ci.TRAIN_GRID)) == 4 * 2 * 2 * 2
    assert len(ci.grid_cases(ci.INFERENCE_GRID)) == 2 * 2 * 2 * 2 * 2
    try:
        ci.create_inference_inputs(device="cpu", fused_normalizer=True)
    except ValueError as e:
        assert "sum_of_keys" in str(e)
    else:
        raise AssertionError("fused_normalizer must be refused")
