"""The reference's own test tables for the two operators (perf/tests/test_list.py:248-259, :274-335),
walked with the package's input factories: shape / dtype / device contracts of outputs and gradients
(perf/tests/common_tests.py:24-62) and agreement with the fp32 oracle on the same seeded inputs."""
import pytest
import torch

from oracle import power_retention_oracle as oracle
from retention_integration_b200 import create_inputs as ci
from tests._golden import make_state, rel_l2

pytestmark = pytest.mark.gpu


def _id(kw):
    return "-".join(f"{k}{v}" for k, v in kw.items() if k in ("t", "tq", "tk", "d", "qhead_ratio", "gating",
                                                               "chunk_size", "initial_state", "switch_over_seq_len"))


@pytest.mark.parametrize("kw", ci.grid_cases(ci.TRAIN_GRID), ids=_id)
def test_training_grid(cuda_device, kw):
    import retention_integration_b200 as prb

    inputs = ci.create_inputs(device=cuda_device, requires_grad=True, **kw)
    Y = prb.power_retention(**inputs)
    (shape, dtype, _), = ci.output_properties(**kw).values()
    assert tuple(Y.shape) == shape and Y.dtype == dtype and Y.is_cuda
    torch.manual_seed(7)
    dY = torch.randn_like(Y)
    Y.backward(dY)
    for name, (shape, dtype, _) in ci.input_properties(**kw).items():
        g = inputs[name].grad
        assert g is not None and tuple(g.shape) == shape and g.dtype == dtype, name
    ref_in = {k: (v.detach().float().cpu().requires_grad_(True) if torch.is_tensor(v) else v) for k, v in inputs.items()}
    Y_ref = oracle.power_retention(**ref_in)
    Y_ref.backward(dY.float().cpu())
    assert rel_l2(Y.float().cpu(), Y_ref) < 2e-2
    for name in ci.input_properties(**kw):
        assert rel_l2(inputs[name].grad.float().cpu(), ref_in[name].grad) < 2e-2, name


@pytest.mark.parametrize("kw", ci.grid_cases(ci.INFERENCE_GRID) + ci.grid_cases(ci.INFERENCE_GRID_NO_CACHE), ids=_id)
def test_inference_grid(cuda_device, kw):
    import retention_integration_b200 as prb
    from retention_integration_b200 import layout

    inputs = ci.create_inference_inputs(device=cuda_device, **kw)
    if inputs["initial_state"] is not None:
        # the factory's state is white noise (a shape contract); for values to compare, a state that real keys
        # and values leave behind: its normaliser is positive
        st, sk = make_state(kw["b"], kw["h"], kw["d"], 32, torch.Generator().manual_seed(3))
        inputs["initial_state"], inputs["sum_of_keys"] = (st / kw["d"]).bfloat16().to(cuda_device), (sk / kw["d"]).to(cuda_device)
    Y, state, sok = prb.power_retention_inference(**inputs)
    want = ci.inference_output_properties(**kw)
    for name, got in (("Y", Y), ("state", state), ("sum_of_keys", sok)):
        if want[name] is None:
            assert got is None, name
        else:
            assert tuple(got.shape) == want[name][0] and got.dtype == want[name][1], name
    d = kw["d"]
    ref_in = {k: (v.detach().float().cpu() if torch.is_tensor(v) else v) for k, v in inputs.items()}
    if ref_in["initial_state"] is not None:
        ref_in["initial_state"] = layout.to_reference_layout(ref_in["initial_state"], d)
        ref_in["sum_of_keys"] = layout.to_reference_layout(ref_in["sum_of_keys"], d, dim=-1)
    Y_ref, st_ref, sk_ref = oracle.power_retention_inference(**ref_in)
    assert rel_l2(Y.float().cpu(), Y_ref) < 1e-2
    if kw["tk"] >= kw.get("switch_over_seq_len", 1 << 30):
        assert rel_l2(state.float().cpu(), layout.from_reference_layout(st_ref, d)) < 1e-2
        assert rel_l2(sok.cpu(), layout.from_reference_layout(sk_ref, d, dim=-1)) < 5e-3
