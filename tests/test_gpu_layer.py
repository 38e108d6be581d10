"""Whole-layer parity on the GPU (fmoe_layer_forward behind the FlashMoE module)."""

import os

import numpy as np
import pytest
import torch

from oracle import flashmoe_oracle as O
from tests.helpers import bf16_ulp_close, make_layer_pair, randn

pytestmark = pytest.mark.gpu


def run_layer(ours, x, **kw):
    from flash_moe_b200 import check_status

    with torch.no_grad():
        y, logits = ours(x.cuda(), return_routing=True, **kw)
    torch.cuda.synchronize()
    check_status()
    return y.cpu(), logits.cpu(), ours.last_indices.cpu(), ours.last_gates.cpu()


def chained_checks(ref, x, y, logits, idx, gates, dtype, out_tol, strict=True):
    """The parity chain: our logits vs fp32, the reference routing applied to OUR logits, and the
    outputs vs an fp32 evaluation teacher-forced on our indices and gates."""
    T = x.shape[0] * x.shape[1]
    nk, k = ref.num_keys, ref.top_k
    x2 = x.reshape(T, -1)
    with torch.no_grad():
        bn = ref.router_norm
        want_logits, _ = O.router_front(
            x2.float(), ref.router_gate.weight.float(),
            bn.running_mean.float().clone(), bn.running_var.float().clone(), False,
        )
        lg = logits.transpose(0, 1).reshape(T, 2 * nk)
        assert O.rel_rms_error(lg.float(), want_logits) < (2e-2 if dtype != torch.float32 else 1e-4)
        # reference routing on our logits
        lp = torch.log_softmax(logits.float(), dim=-1).to(dtype).contiguous()
        want_s, want_i = O.router_topk(lp, nk, k)
        viol = O.check_router_threshold(lp, nk, k, idx, rel=1e-3 if dtype == torch.float32 else 8e-3)
        assert all(v == 0 for v in viol.values()), viol
        same = (torch.sort(idx, -1).values == torch.sort(want_i, -1).values).all(-1).float().mean().item()
        assert same > (0.999 if dtype == torch.float32 else 0.97), same
        want_g = O.routing_weights(want_s, ref.norm_topk_prob)
        rows = (idx == want_i).all(-1)
        if dtype == torch.float32:
            torch.testing.assert_close(gates[rows], want_g[rows], rtol=1e-4, atol=1e-7)
        else:
            assert bf16_ulp_close(gates[rows], want_g[rows], 2).all()
        want_y = ref.forward_fp32_given_routing(x, idx, gates)
        want_y_h = ref.forward_fp32_given_routing(x, idx, gates, round_h_to=None if dtype == torch.float32 else dtype)
    # gate 1: against the evaluation that, like every 16-bit pipeline, stores the MLP intermediate in
    # the module dtype - nothing but the final rounding (+3e-3) may remain (`strict`, the default)
    O.assert_output_parity(y, want_y_h, dtype, raw_budget=out_tol, strict=strict)
    # gate 2: against the pure float32 evaluation (budget 2e-2 x RMS, or the rounding floor of the
    # output format plus the 8e-3 that the 16-bit intermediate can cost)
    return O.assert_output_parity(y, want_y, dtype, raw_budget=out_tol)


def test_layer_config1_fp32_matches_reference_fixture(golden_dir):
    """Benchmark configuration 1 (T=256, H=256, I=1024, N=1024, k=8, fp32): against the output the
    reference's eager module produced for the same seeds."""
    z = np.load(os.path.join(golden_dir, "eager_c1_fp32.npz"))
    ref, ours = make_layer_pair(256, 1024, 1024, 8, False, torch.float32)
    ref.eval(); ours.eval()
    x = torch.randn(1, 256, 256, generator=torch.Generator().manual_seed(1))
    y, logits, idx, gates = run_layer(ours, x)
    np.testing.assert_allclose(logits.contiguous().numpy(), z["router_logits"], rtol=1e-4, atol=2e-5)
    same = (np.sort(idx.numpy(), -1) == np.sort(z["indices"], -1)).all(-1).mean()
    assert same > 0.99
    rms = float(np.sqrt((z["y"] ** 2).mean()))
    rows = (np.sort(idx.numpy(), -1) == np.sort(z["indices"], -1)).all(-1)
    assert np.abs(y.numpy()[0][rows] - z["y"][0][rows]).max() < 1e-3 * rms
    chained_checks(ref, x, y, logits, idx, gates, torch.float32, 1e-4)


@pytest.mark.parametrize(
    "H,I,N,k,norm,B,S",
    [(256, 1024, 1024, 8, False, 1, 256), (512, 768, 4096, 16, True, 2, 192), (128, 256, 256, 4, False, 3, 50),
     (1024, 4096, 16384, 64, False, 1, 512),
     # ragged for the CTA-pair GEMMs: 777 rows (not a multiple of 128), 520 output columns (not a multiple of 32, so
     # the last box of the epilogue's addend tile hangs over the edge), 536 intermediate columns
     (520, 536, 1024, 8, False, 1, 777)],
)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_layer_16bit_chained_parity(H, I, N, k, norm, B, S, dtype):
    ref, ours = make_layer_pair(H, I, N, k, norm, dtype)
    ref.eval(); ours.eval()
    x = randn((B, S, H), 1, dtype)
    y, logits, idx, gates = run_layer(ours, x)
    chained_checks(ref, x, y, logits, idx, gates, dtype, 2e-2)
    y2, *_ = run_layer(ours, x)
    assert torch.equal(y, y2)


def test_layer_train_mode_batch_statistics():
    ref, ours = make_layer_pair(256, 512, 1024, 8, True, torch.float32)
    ref.train(); ours.train()
    x = randn((2, 128, 256), 3) * 1.5 + 0.3
    with torch.no_grad():
        want_y, want_logits = ref(x)
    y, logits, idx, gates = run_layer(ours, x)
    torch.testing.assert_close(logits.contiguous(), want_logits.contiguous(), rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(ours.router_norm.running_mean.cpu(), ref.router_norm.running_mean, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(ours.router_norm.running_var.cpu(), ref.router_norm.running_var, rtol=1e-4, atol=1e-6)
    assert int(ours.router_norm.num_batches_tracked) == 1


def test_layer_config2_full_size_bf16():
    """Benchmark configuration 2 (T=4096, H=1024, I=4096, N=16384, k=64, bf16), teacher-forced output parity and
    the same result with the shared MLP on the main stream."""
    ref, ours = make_layer_pair(1024, 4096, 16384, 64, False, torch.bfloat16)
    ref.eval(); ours.eval()
    x = randn((1, 4096, 1024), 1, torch.bfloat16)
    y, logits, idx, gates = run_layer(ours, x)
    err = chained_checks(ref, x, y, logits, idx, gates, torch.bfloat16, 2e-2, strict=True)
    print("config 2 teacher-forced error / RMS:", err)
    ours.overlap_shared_mlp = False
    y2, *_ = run_layer(ours, x)
    assert torch.equal(y, y2)


def test_state_dict_and_device_contract():
    from flash_moe_b200 import FlashMoE, FlashMoEConfig

    ref, ours = make_layer_pair(128, 256, 256, 4, False, torch.bfloat16)
    assert set(ref.state_dict()) == set(ours.state_dict())
    other = FlashMoE(FlashMoEConfig(128, 256, "silu", 256, 4)).to(torch.bfloat16).cuda()
    other.load_state_dict(ref.state_dict())
    x = randn((1, 64, 128), 2, torch.bfloat16).cuda()
    ours.eval(); other.eval()
    assert torch.equal(ours(x)[0], other(x)[0])
    with pytest.raises(Exception):
        ours(x.cpu())


def test_cuda_graph_replay_matches_eager():
    from flash_moe_b200 import GraphedFlashMoE, check_status

    ref, ours = make_layer_pair(256, 512, 1024, 8, True, torch.bfloat16)
    ours.eval()
    x = randn((2, 96, 256), 4, torch.bfloat16).cuda()
    with torch.no_grad():
        y, logits = ours(x)
        g = GraphedFlashMoE(ours, x)
        y2, logits2 = (t.clone() for t in g(x))  # the static outputs are overwritten by the next replay
        x3 = randn((2, 96, 256), 5, torch.bfloat16).cuda()
        y3, _ = g(x3)
        want3, _ = ours(x3)
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(y, y2) and torch.equal(logits, logits2)
    assert torch.equal(y3, want3)


def test_launch_and_candidate_switches_do_not_change_results(monkeypatch):
    """Programmatic dependent launch only changes when a kernel may start, and the top-k's register-resident
    candidate list only where the candidates live: the layer's outputs are bit-equal with either switched off, at a
    small shape and at the benchmark's (the one that uses the 10-per-lane candidate registers)."""
    from flash_moe_b200 import check_status

    for (H, I, N, k, shape) in ((256, 512, 1024, 8, (2, 96, 256)), (1024, 4096, 16384, 64, (1, 1024, 1024))):
        _, ours = make_layer_pair(H, I, N, k, False, torch.bfloat16)
        ours.eval()
        x = randn(shape, 4, torch.bfloat16).cuda()
        with torch.no_grad():
            monkeypatch.delenv("FMOE_PDL", raising=False)
            monkeypatch.delenv("FMOE_TOPK_CANDIDATES", raising=False)
            y, logits = ours(x)
            monkeypatch.setenv("FMOE_PDL", "0")
            y_plain, logits_plain = ours(x)
            monkeypatch.setenv("FMOE_PDL", "31")
            y_all, _ = ours(x)
            monkeypatch.delenv("FMOE_PDL")
            monkeypatch.setenv("FMOE_TOPK_CANDIDATES", "smem")
            y_smem, _ = ours(x)
        torch.cuda.synchronize()
        check_status()
        assert torch.equal(y, y_plain) and torch.equal(logits, logits_plain)
        assert torch.equal(y, y_all) and torch.equal(y, y_smem)


def test_stage_events_cover_the_forward():
    """The library records an event pair per stage (enum fmoe_stage); the stages follow one another on the stream."""
    from flash_moe_b200 import StageTimer, _lib

    ref, ours = make_layer_pair(256, 512, 1024, 8, False, torch.bfloat16)
    ours.eval()
    x = randn((1, 512, 256), 6, torch.bfloat16).cuda()
    timer = StageTimer()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.no_grad():
        ours(x)
        start.record()
        y, _ = ours(x, stage_timer=timer)
        end.record()
        want, _ = ours(x)
    torch.cuda.synchronize()
    ms = timer.elapsed_ms()
    assert tuple(ms) == _lib.STAGE_NAMES and len(ms) == 6
    assert all(v > 0 for v in ms.values())
    assert sum(ms.values()) <= start.elapsed_time(end) * 1.05
    ev = timer.events  # end of one stage is not after the start of the next
    for i in range(5):
        assert ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) >= 0
    assert torch.equal(y, want)


def test_graph_keeps_its_workspace_when_the_layer_outgrows_it():
    """A captured graph has the layer's scratch addresses baked in.  A later eager forward with more tokens makes the
    layer allocate a larger workspace; the graph must keep (and keep using) the one it was captured with."""
    from flash_moe_b200 import GraphedFlashMoE, check_status

    ref, ours = make_layer_pair(256, 512, 1024, 8, False, torch.bfloat16)
    ours.eval()
    small = randn((1, 64, 256), 21, torch.bfloat16).cuda()
    big = randn((4, 512, 256), 22, torch.bfloat16).cuda()
    with torch.no_grad():
        g = GraphedFlashMoE(ours, small)
        want, _ = (t.clone() for t in g(small))
        ws_before = {k: v.data_ptr() for k, v in ours._workspaces.items()}
        ours(big)  # grows (replaces) the layer's own workspace
        assert any(ours._workspaces[k].data_ptr() != p for k, p in ws_before.items())
        junk = [torch.full((1 << 22,), 7, dtype=torch.uint8, device="cuda") for _ in range(8)]  # would land in freed memory
        got, _ = g(small)
        eager, _ = ours(small)
    torch.cuda.synchronize()
    check_status()
    del junk
    assert torch.equal(got, want) and torch.equal(got, eager)


def test_residual_is_added_before_the_single_rounding():
    from flash_moe_b200 import check_status

    ref, ours = make_layer_pair(256, 512, 1024, 8, False, torch.bfloat16)
    ours.eval()
    for shape in ((1, 96, 256), (2, 300, 256)):  # one-CTA and CTA-pair down GEMM
        x = randn(shape, 23, torch.bfloat16).cuda()
        r = (randn(shape, 24, torch.bfloat16) * 3).cuda()
        with torch.no_grad():
            y, logits = ours(x)
            z, logits_r = ours(x, residual=r)
        torch.cuda.synchronize()
        check_status()
        assert torch.equal(logits, logits_r)
        tol = 2.0 ** -7 * torch.maximum(y.float().abs(), z.float().abs()) + 1e-6
        assert ((z.float() - (r.float() + y.float())).abs() <= tol).all()
    with pytest.raises(Exception):
        ours(x, residual=r[:, :-1])
    # float32 module: the CUDA-core GEMM path takes the residual too
    ref32, ours32 = make_layer_pair(128, 256, 256, 4, False, torch.float32)
    ours32.eval()
    x = randn((1, 80, 128), 25, torch.float32).cuda()
    r = randn((1, 80, 128), 26, torch.float32).cuda()
    with torch.no_grad():
        torch.testing.assert_close(ours32(x, residual=r)[0], r + ours32(x)[0], rtol=1e-5, atol=1e-5)


def test_stack_replays_from_one_graph():
    """Eight-layer-style residual stack (here three layers) captured in ONE CUDA graph: replay equals eager."""
    from flash_moe_b200 import FlashMoEConfig, GraphedFlashMoE, check_status
    from flash_moe_b200.modules.stack import FlashMoEStack

    stack = FlashMoEStack(FlashMoEConfig(256, 512, "silu", 1024, 8, True), 3, seeds=[0, 1, 2]).to(torch.bfloat16).eval().cuda()
    x = (randn((2, 200, 256), 27, torch.bfloat16) * 0.5).cuda()
    x2 = (randn((2, 200, 256), 28, torch.bfloat16) * 0.5).cuda()
    with torch.no_grad():
        want, want_logits = stack(x)
        g = GraphedFlashMoE(stack, x)
        got, got_logits = g(x)
        got = got.clone()
        got_logits = [t.clone() for t in got_logits]
        got2 = g(x2)[0].clone()
        want2, _ = stack(x2)
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(got, want) and torch.equal(got2, want2)
    assert all(torch.equal(a, b) for a, b in zip(got_logits, want_logits))


def test_bounded_wait_gives_up_and_the_context_survives():
    """The give-up path of the device-side waits: a kernel waits ~1 ms on a barrier nothing completes, reports
    FMOE_STATUS_WAIT_TIMEOUT and returns; the next launches work."""
    from flash_moe_b200 import _lib, check_status

    dev = torch.device("cuda", 0)
    _lib.read_status(dev)
    result = torch.zeros(1, dtype=torch.int32, device=dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    rc = _lib.lib().fmoe_selftest_wait_timeout(1_000_000, _lib.status_word(dev).data_ptr(), result.data_ptr(),
                                               _lib.current_stream_ptr(dev))
    b.record()
    assert rc == 0
    torch.cuda.synchronize()
    assert 0.5 < a.elapsed_time(b) < 50.0  # gave up after about a millisecond, not after the 2 s default
    assert int(result.item()) == 2
    with pytest.raises(_lib.FmoeError, match="timed out"):
        check_status(dev)
    assert _lib.read_status(dev) == 0  # cleared by the read above
    ref, ours = make_layer_pair(128, 256, 256, 4, False, torch.bfloat16)
    ours.eval()
    x = randn((1, 64, 128), 29, torch.bfloat16).cuda()
    with torch.no_grad():
        y, _ = ours(x)
    torch.cuda.synchronize()
    check_status(dev)
    assert torch.isfinite(y.float()).all()


def test_batch_norm_edge_cases_follow_torch():
    """momentum=None is torch's cumulative moving average (factor 1 / batches seen); a one-row training batch raises."""
    import torch.nn as nn

    ref, ours = make_layer_pair(128, 256, 256, 4, False, torch.float32)
    ours.train()
    ours.router_norm.momentum = None
    bn = nn.BatchNorm1d(128, affine=False, momentum=None)
    xs = [randn((1, 96, 128), 40 + i) * (1.0 + 0.3 * i) + 0.2 * i for i in range(3)]
    with torch.no_grad():
        for x in xs:
            ours(x.cuda())
            bn(x.view(-1, 128))
    torch.testing.assert_close(ours.router_norm.running_mean.cpu(), bn.running_mean, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(ours.router_norm.running_var.cpu(), bn.running_var, rtol=1e-4, atol=1e-6)
    assert int(ours.router_norm.num_batches_tracked) == 3
    with pytest.raises(ValueError, match="more than 1 value per channel"):
        with torch.no_grad():
            ours(randn((1, 1, 128), 50).cuda())


def test_pre_norm_stack_matches_torch_composition():
    """Pre-norm decoder composition x <- x + layer(rms_norm(x)): the library's norm kernel against torch's, the stack
    against the same steps written out by hand, and the whole thing replayed from one graph."""
    import torch.nn.functional as F

    from flash_moe_b200 import FlashMoEConfig, GraphedFlashMoE, check_status
    from flash_moe_b200.modules.stack import FlashMoEStack
    from flash_moe_b200.ops.rms_norm import rms_norm

    for dt in (torch.bfloat16, torch.float32):
        x = (randn((3, 50, 256), 60, dt) * 2.0).cuda()
        w = (randn((256,), 61, dt) * 0.1 + 1.0).cuda()
        want = F.rms_norm(x.float(), (256,), w.float(), 1e-6)
        got = rms_norm(x, w, 1e-6)
        if dt == torch.float32:
            torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
        else:
            assert bf16_ulp_close(got.cpu(), want.to(dt).cpu(), 1).all()
        if dt == torch.bfloat16:  # without a weight
            assert bf16_ulp_close(rms_norm(x, None).cpu(), F.rms_norm(x.float(), (256,), None, 1e-6).to(dt).cpu(), 1).all()
    stack = FlashMoEStack(FlashMoEConfig(256, 512, "silu", 1024, 8, True), 3, seeds=[0, 1, 2], pre_norm=True)
    stack = stack.to(torch.bfloat16).eval().cuda()
    with torch.no_grad():
        for i, p in enumerate(stack.norms):
            p.copy_((randn((256,), 70 + i, torch.bfloat16) * 0.1 + 1.0).cuda())
        x = (randn((2, 200, 256), 62, torch.bfloat16) * 3.0).cuda()
        cur = x
        for i, layer in enumerate(stack.layers):
            cur, _ = layer(rms_norm(cur, stack.norms[i], stack.norm_eps), residual=cur)
        got, _ = stack(x)
        g = GraphedFlashMoE(stack, x)
        replayed = g(x)[0].clone()
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(got, cur) and torch.equal(replayed, got)
    assert torch.isfinite(got.float()).all()
