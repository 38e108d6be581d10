"""Expert and shared-MLP parity on the GPU through the C ABI (fmoe_expert_forward / fmoe_mlp_forward)."""

import os

import numpy as np
import pytest
import torch

from oracle import flashmoe_oracle as O
from tests.helpers import randn

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2  # max |err| / RMS(oracle), the layer-output budget for 16-bit results
F32_TOL = 2e-5


def expert_inputs(T, H, N, k, dtype, seed=0, zipf=False):
    x = randn((T, H), seed + 1, dtype, 0.5)
    d = randn((N, H), seed + 2, dtype, 0.1)
    u = randn((N, H), seed + 3, dtype, 0.1)
    g = torch.Generator().manual_seed(seed + 4)
    if zipf:
        p = torch.arange(1, N + 1, dtype=torch.float64).pow(-1.1)
        cdf = torch.cumsum(p / p.sum(), 0)
        idx = torch.searchsorted(cdf, torch.rand(T, k, generator=g, dtype=torch.float64)).clamp_(max=N - 1)
    else:
        idx = torch.randint(0, N, (T, k), generator=g)
    gates = torch.softmax(torch.randn(T, k, generator=g), dim=-1).to(dtype)
    return x, d, u, idx, gates


@pytest.mark.parametrize(
    "T,H,N,k",
    [(64, 256, 1024, 8), (300, 1024, 4096, 16), (17, 72, 50, 3), (128, 2048, 512, 4), (33, 4096, 64, 2),
     (256, 512, 7, 5), (1, 128, 16, 1)],
)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_expert_forward(T, H, N, k, dtype):
    from flash_moe_b200 import check_status
    from flash_moe_b200.ops.flash_expert import flash_expert_fp32, flash_expert_func

    if dtype == torch.float32 and H % 4:
        pytest.skip("row size must be a multiple of 16 bytes")
    x, d, u, idx, gates = expert_inputs(T, H, N, k, dtype, seed=T + H)
    idx[0, -1] = idx[0, 0]  # duplicate expert inside a token accumulates
    want = O.expert_forward(x, d, u, idx, gates)
    got = flash_expert_func(x.cuda(), d.cuda(), u.cuda(), idx.cuda(), gates.cuda())
    acc = flash_expert_fp32(x.cuda(), d.cuda(), u.cuda(), idx.cuda(), gates.cuda())
    again = flash_expert_func(x.cuda(), d.cuda(), u.cuda(), idx.cuda(), gates.cuda())
    check_status()
    assert got.dtype == dtype and acc.dtype == torch.float32
    assert O.rel_rms_error(acc.cpu(), want) < F32_TOL * 10
    O.assert_output_parity(got.cpu(), want, dtype)
    assert torch.equal(got, again), "the expert path must be run-to-run deterministic"


def test_expert_zipf_hot_expert_and_empty_experts():
    from flash_moe_b200.ops.flash_expert import flash_expert_fp32

    T, H, N, k = 512, 256, 65536, 16
    x, d, u, idx, gates = expert_inputs(T, H, N, k, torch.bfloat16, seed=9, zipf=True)
    assert torch.bincount(idx.flatten(), minlength=N).max() > 200  # one expert owns many pairs
    want = O.expert_forward(x, d, u, idx, gates)
    got = flash_expert_fp32(x.cuda(), d.cuda(), u.cuda(), idx.cuda(), gates.cuda())
    assert O.rel_rms_error(got.cpu(), want) < 1e-4
    idx[:] = 3  # every pair on one expert
    want = O.expert_forward(x, d, u, idx, gates)
    got = flash_expert_fp32(x.cuda(), d.cuda(), u.cuda(), idx.cuda(), gates.cuda())
    assert O.rel_rms_error(got.cpu(), want) < 1e-4


def test_expert_out_of_range_ids_are_skipped_and_flagged():
    from flash_moe_b200 import read_status
    from flash_moe_b200.ops.flash_expert import flash_expert_fp32

    T, H, N, k = 32, 128, 64, 4
    x, d, u, idx, gates = expert_inputs(T, H, N, k, torch.bfloat16, seed=2)
    read_status()
    bad = idx.clone()
    bad[3, 1] = N
    bad[5, 0] = -1
    got = flash_expert_fp32(x.cuda(), d.cuda(), u.cuda(), bad.cuda(), gates.cuda())
    assert read_status() & 1
    g2 = gates.clone()
    g2[3, 1] = 0
    g2[5, 0] = 0
    want = O.expert_forward(x, d, u, bad.clamp(0, N - 1), g2)
    assert O.rel_rms_error(got.cpu(), want) < 1e-4
    assert read_status() == 0
    # -1 alone is the empty-slot value: skipped without raising the flag, in both dtypes' schedules
    for dtype in (torch.bfloat16, torch.float32):
        x, d, u, idx, gates = expert_inputs(T, H, N, k, dtype, seed=2)
        empty = idx.clone()
        empty[5, 0] = -1
        empty[7, :] = -1
        got = flash_expert_fp32(x.cuda(), d.cuda(), u.cuda(), empty.cuda(), gates.cuda())
        assert read_status() == 0
        g2 = gates.clone()
        g2[empty == -1] = 0
        assert O.rel_rms_error(got.cpu(), O.expert_forward(x, d, u, empty.clamp(0, N - 1), g2)) < 1e-4
        assert float(got[7].abs().max()) == 0.0


def test_expert_matches_reference_kernel_fixture(golden_dir):
    from flash_moe_b200.ops.flash_expert import flash_expert_func

    z = np.load(os.path.join(golden_dir, "triton_expert_small.npz"))
    t = {n: torch.from_numpy(z[n]).cuda() for n in z.files}
    got = flash_expert_func(t["x"], t["down"], t["up"], t["indices"], t["gates"])
    np.testing.assert_allclose(got.cpu().numpy(), z["y"], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize(
    "T,H,I", [(256, 256, 1024), (200, 136, 264), (128, 1024, 4096), (1000, 512, 384), (3, 64, 128), (129, 128, 8)]
)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_mlp_forward(T, H, I, dtype):
    from flash_moe_b200 import check_status
    from flash_moe_b200.ops.flash_mlp import flash_mlp_add, flash_mlp_func

    x = randn((T, H), 1, dtype, 0.5)
    wg = randn((I, H), 2, dtype, 1.0 / H**0.5)
    wu = randn((I, H), 3, dtype, 1.0 / H**0.5)
    wd = randn((H, I), 4, dtype, 1.0 / I**0.5)
    add = randn((T, H), 5, torch.float32, 0.3)
    # 16-bit: the intermediate h lives in the storage dtype between the two GEMMs (as in the reference)
    want = O.mlp_forward(x, wg, wu, wd, round_h_to=None if dtype == torch.float32 else dtype)
    got = flash_mlp_func(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda())
    got_add = flash_mlp_add(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda(), add.cuda())
    again = flash_mlp_func(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda())
    check_status()
    O.assert_output_parity(got.cpu(), want, dtype, strict=True)
    O.assert_output_parity(got_add.cpu(), want + add, dtype, strict=True)
    assert torch.equal(got, again)


def test_mlp_matches_reference_kernel_fixture(golden_dir):
    from flash_moe_b200.ops.flash_mlp import flash_mlp_func

    z = np.load(os.path.join(golden_dir, "triton_mlp_small.npz"))
    t = {n: torch.from_numpy(z[n]).cuda() for n in z.files}
    got = flash_mlp_func(t["x"], t["wg"], t["wu"], t["wd"])
    np.testing.assert_allclose(got.cpu().numpy(), z["y"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("T,H,G", [(1, 4, 1), (37, 64, 3), (513, 2048, 8)])
def test_combine_partial_rows_sums_in_source_order(T, H, G):
    """fmoe_combine_partial_rows: out[t] = sum_g rows[slot[g, t]] in float32, ascending g, -1 skipped - bit exact."""
    from flash_moe_b200 import check_status
    from flash_moe_b200.ops.flash_expert import combine_partial_rows

    g = torch.Generator().manual_seed(T + H)
    present = torch.rand(G, T, generator=g) < 0.6
    R = int(present.sum())
    slot = torch.full((G, T), -1, dtype=torch.int32)
    slot[present] = torch.randperm(R, generator=g).to(torch.int32)
    rows = torch.randn(R + 3, H, generator=g)  # three rows nobody points at
    want = torch.zeros(T, H)
    for s in range(G):
        m = slot[s] >= 0
        want[m] = want[m] + rows[slot[s][m].long()]
    got = combine_partial_rows(rows.cuda(), slot.cuda(), T)
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(got.cpu(), want)
    with pytest.raises(Exception):
        combine_partial_rows(rows.cuda().to(torch.bfloat16), slot.cuda(), T)


def test_gather_roof_probe_runs_and_rejects_bad_rows():
    from flash_moe_b200 import _lib
    from flash_moe_b200.bench_gather_roof import measure_gather_roof

    best, per_grid = measure_gather_roof("cuda:0", row_bytes=1024, rows=4096, count=65536, reps=2)
    assert best > 100.0 and len(per_grid) == 6  # GB/s; any working GPU is far above this
    assert per_grid["bulk_ring"] > 100.0 and per_grid["cp_async_ring"] > 100.0
    _lib.read_status()
    t = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    L, st, stream = _lib.lib(), _lib.status_word(t.device).data_ptr(), _lib.current_stream_ptr(t.device)
    rc = L.fmoe_gather_probe(t.data_ptr(), 4, ids.data_ptr(), 8, 768, 4, 0, None, st, stream)
    assert rc == 4  # FMOE_ERR_ALIGNMENT: register-load rows must be multiples of 512 bytes
    # a row id outside the table is not followed: row 0 is read instead and the status word says so
    for mode in (0, 1, 2):
        ids = torch.tensor([0, 1, 2, 3, 1 << 20, -5, 2, 1], dtype=torch.int32, device="cuda")
        assert L.fmoe_gather_probe(t.data_ptr(), 8, ids.data_ptr(), 8, 512, 4, mode, None, st, stream) == 0
        assert _lib.read_status() == _lib.STATUS_BAD_ROW_INDEX
        ids = torch.tensor([0, 1, 2, 3, 7, 6, 2, 1], dtype=torch.int32, device="cuda")
        assert L.fmoe_gather_probe(t.data_ptr(), 8, ids.data_ptr(), 8, 512, 4, mode, None, st, stream) == 0
        assert _lib.read_status() == 0


def test_empty_inputs():
    """No tokens, or no experts per token: empty / zero results, no launch errors."""
    from flash_moe_b200 import FlashMoE, FlashMoEConfig, check_status
    from flash_moe_b200.ops.flash_expert import flash_expert_func
    from flash_moe_b200.ops.flash_mlp import flash_mlp_func
    from flash_moe_b200.ops.pkm import pkm_func

    dt = torch.bfloat16
    d, u = randn((32, 64), 1, dt).cuda(), randn((32, 64), 2, dt).cuda()
    x0 = torch.empty(0, 64, dtype=dt, device="cuda")
    idx0 = torch.empty(0, 4, dtype=torch.int64, device="cuda")
    assert flash_expert_func(x0, d, u, idx0, torch.empty(0, 4, dtype=dt, device="cuda")).shape == (0, 64)
    x = randn((5, 64), 3, dt).cuda()
    none = flash_expert_func(x, d, u, torch.empty(5, 0, dtype=torch.int64, device="cuda"), torch.empty(5, 0, dtype=dt, device="cuda"))
    assert none.shape == (5, 64) and float(none.abs().max()) == 0.0
    assert float(pkm_func(u, torch.empty(5, 0, dtype=dt, device="cuda"), torch.empty(5, 0, dtype=torch.int64, device="cuda")).abs().max()) == 0.0
    wg, wu, wd = randn((128, 64), 4, dt).cuda(), randn((128, 64), 5, dt).cuda(), randn((64, 128), 6, dt).cuda()
    assert flash_mlp_func(x0, wg, wu, wd).shape == (0, 64)
    layer = FlashMoE(FlashMoEConfig(64, 128, "silu", 64, 4)).to(dt).cuda().eval()
    with torch.no_grad():
        y, logits = layer(torch.empty(1, 0, 64, dtype=dt, device="cuda"))
    assert y.shape == (1, 0, 64) and logits.shape == (2, 0, 8)
    torch.cuda.synchronize()
    check_status()
