"""The CPU oracle against the fixtures produced by the reference's own code (tests/golden/make_golden.py)."""

import os

import numpy as np
import pytest
import torch

from oracle import flashmoe_oracle as O

DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16}


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


def build_oracle_layer(z, with_params):
    H, I, N, k, norm, B, S, train = [int(v) for v in z["cfg"]]
    dtype = DT[str(z["dtype"])]
    torch.manual_seed(0)
    m = O.OracleFlashMoE(H, I, N, k, bool(norm))
    if with_params:
        sd = {n[len("param."):]: torch.from_numpy(z[n]) for n in z.files if n.startswith("param.")}
        m.load_state_dict(sd)
        x = torch.from_numpy(z["x"])
    else:
        x = torch.randn(B, S, H, generator=torch.Generator().manual_seed(1))
    m = m.to(dtype)
    m.train(bool(train))
    return m, x.to(dtype)


@pytest.mark.parametrize("name", ["eager_mini_fp32", "eager_mini_fp32_train_norm", "eager_c1_fp32"])
def test_layer_fp32_matches_reference_eager(golden_dir, name):
    z = load(golden_dir, name)
    m, x = build_oracle_layer(z, with_params="x" in z.files)
    with torch.no_grad():
        y, logits = m(x)
    # same torch kernels in the same order: logits and batch-norm side effects are bit-equal
    assert np.array_equal(logits.contiguous().numpy(), z["router_logits"])
    assert np.array_equal(m.router_norm.running_mean.numpy(), z["running_mean_after"])
    assert np.array_equal(m.router_norm.running_var.numpy(), z["running_var_after"])
    np.testing.assert_allclose(y.numpy(), z["y"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", ["eager_mini_fp32", "eager_c1_fp32", "eager_mini_bf16"])
def test_routing_matches_reference_eager(golden_dir, name):
    z = load(golden_dir, name)
    dtype = DT[str(z["dtype"])]
    nk = int(np.floor(np.sqrt(int(z["cfg"][2]))))
    k = int(z["cfg"][3])
    lp = torch.from_numpy(z["log_probs"]).to(dtype)
    s, i = O.router_topk(lp, nk, k)
    # the descending score sequence is unique whatever the tie-break
    assert np.array_equal(s.float().numpy(), z["scores"])
    ref_i = torch.from_numpy(z["indices"])
    assert all(v == 0 for v in O.check_router_threshold(lp, nk, k, ref_i, rel=0.0).values())
    if dtype == torch.float32:
        assert torch.equal(i, ref_i)


def test_bf16_eager_layer_close(golden_dir):
    z = load(golden_dir, "eager_mini_bf16")
    m, x = build_oracle_layer(z, with_params=True)
    with torch.no_grad():
        y, logits = m(x)
    assert np.array_equal(logits.contiguous().float().numpy(), z["router_logits"])
    # routing ties may resolve differently (torch.topk vs lowest-index); compare through the fp32 evaluator
    idx = torch.from_numpy(z["indices"])
    gates = O.routing_weights(torch.from_numpy(z["scores"]).to(torch.bfloat16), False)
    with torch.no_grad():
        want = m.forward_fp32_given_routing(x, idx, gates)
    assert O.rel_rms_error(torch.from_numpy(z["y"]), want) < 5e-2


@pytest.mark.parametrize(
    "name", ["triton_router_nk16_k4", "triton_router_nk16_k4_tied", "triton_router_nk32_k8_tied", "triton_router_nk128_k16"]
)
def test_router_matches_reference_triton_kernel(golden_dir, name):
    z = load(golden_dir, name)
    lp = torch.from_numpy(z["log_probs"])
    s, i = O.router_topk(lp, int(z["nk"]), int(z["k"]))
    assert np.array_equal(s.numpy(), z["scores"])
    assert np.array_equal(i.numpy(), z["indices"])  # includes the tie order


def test_expert_matches_reference_triton_kernel(golden_dir):
    z = load(golden_dir, "triton_expert_small")
    t = {n: torch.from_numpy(z[n]) for n in z.files}
    y = O.expert_forward(t["x"], t["down"], t["up"], t["indices"], t["gates"])
    np.testing.assert_allclose(y.numpy(), z["y"], rtol=1e-5, atol=1e-6)
    y2 = O.expert_forward_eager(t["x"], t["down"], t["up"], t["indices"], t["gates"])
    np.testing.assert_allclose(y2.numpy(), z["y"], rtol=1e-5, atol=1e-6)


def test_mlp_matches_reference_triton_kernel(golden_dir):
    z = load(golden_dir, "triton_mlp_small")
    t = {n: torch.from_numpy(z[n]) for n in z.files}
    y = O.mlp_forward(t["x"], t["wg"], t["wu"], t["wd"])
    np.testing.assert_allclose(y.numpy(), z["y"], rtol=1e-5, atol=1e-6)


def test_peer_and_pkm_oracles_match_reference_triton_kernels(golden_dir):
    z = np.load(os.path.join(golden_dir, "triton_peer_pkm_small.npz"))
    x, d, u, w, idx = (torch.from_numpy(z[n]) for n in ("x", "down", "up", "weights", "indices"))
    assert torch.allclose(O.peer_forward(x, d, u, w, idx), torch.from_numpy(z["y_peer"]), rtol=1e-4, atol=1e-5)
    assert torch.allclose(O.pkm_forward(u, w, idx), torch.from_numpy(z["y_pkm"]), rtol=1e-5, atol=1e-6)
