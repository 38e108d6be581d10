"""The one-kernel expert forward (rows streamed through a shared-memory ring) against the oracle and against the
two-pass kernels.  The library picks it by itself only for tables of 1 GiB and more; FMOE_EXPERT_SCHEDULE=fused
forces it for any 16-bit shape it supports, and the variable is read once per process, so the cases run in a child
process."""

import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent(
    """
    import os, sys, torch
    sys.path.insert(0, os.environ["FMOE_ROOT"])
    from flash_moe_b200 import _lib, check_status
    from flash_moe_b200.ops.flash_expert import _expert_forward
    from oracle import flashmoe_oracle as O

    def case(T, H, N, k, dtype, seed, bad=False, zipf=False):
        g = torch.Generator().manual_seed(seed)
        x = (torch.randn(T, H, generator=g) * 0.5).to(dtype)
        down = (torch.randn(N, H, generator=g) * 0.1).to(dtype)
        up = (torch.randn(N, H, generator=g) * 0.1).to(dtype)
        if zipf:  # many duplicates inside a token: they must accumulate
            p = torch.arange(1, N + 1, dtype=torch.float64).pow(-1.3)
            idx = torch.multinomial((p / p.sum()).float(), T * k, replacement=True, generator=g).view(T, k)
        else:
            idx = torch.randint(0, N, (T, k), generator=g)
        gates = torch.softmax(torch.randn(T, k, generator=g), -1).to(dtype)
        if bad:
            idx[0, 0] = -1          # empty slot: skipped silently
            idx[1, k - 1] = N + 5   # out of range: skipped and flagged
            idx[2, 0] = -7
        want = O.expert_forward(x.float(), down.float(), up.float(), idx.clamp(0, N - 1), 
                                torch.where((idx >= 0) & (idx < N), gates.float(), torch.zeros(())))
        xd, dd, ud, id_, gd = (t.cuda() for t in (x, down, up, idx, gates))
        got32 = _expert_forward(xd, dd, ud, id_, gd, out_dtype=torch.float32)
        got16, raw = _expert_forward(xd, dd, ud, id_, gd, save_scores=True)
        again = _expert_forward(xd, dd, ud, id_, gd, out_dtype=torch.float32)
        torch.cuda.synchronize()
        status = _lib.read_status()
        assert status == (_lib.STATUS_BAD_EXPERT_ID if bad else 0), status
        assert torch.equal(got32, again), "reruns must be bit-equal"
        rms = want.pow(2).mean().sqrt()
        e32 = float((got32.cpu() - want).abs().max() / rms)
        assert e32 < 2e-4, (T, H, N, k, e32)
        O.assert_output_parity(got16.cpu(), want, dtype)
        s_want = (x.float()[:, None, :] * down.float()[idx.clamp(0, N - 1)]).sum(-1)
        s_want = torch.where((idx >= 0) & (idx < N), s_want, torch.zeros(()))
        assert float((raw.cpu() - s_want).abs().max()) < 1e-3 * max(1.0, float(s_want.abs().max()))
        return got32

    assert os.environ.get("FMOE_EXPERT_SCHEDULE") == "fused"
    bf, hf = torch.bfloat16, torch.float16
    outs = {}
    # (tokens, hidden, experts, slots per token): full groups, ragged last group, several rounds of 64 slots,
    # hidden sizes that are not a multiple of the 256-column steps, the widest supported row
    shapes = [(64, 256, 512, 8, bf), (200, 1024, 2048, 64, bf), (96, 512, 1000, 20, bf), (130, 1000, 777, 70, bf),
              (77, 200, 300, 1, bf), (128, 2048, 4096, 16, bf), (150, 1536, 999, 130, hf), (64, 64, 128, 33, hf)]
    for i, (T, H, N, k, dt) in enumerate(shapes):
        outs[i] = case(T, H, N, k, dt, 100 + i)
    case(90, 768, 500, 24, bf, 300, bad=True)
    case(100, 1024, 64, 48, bf, 301, zipf=True)
    torch.save({i: o.cpu() for i, o in outs.items()}, os.environ["FMOE_OUT"])
    print("fused cases ok")
    """
)

TWO_PASS = textwrap.dedent(
    """
    import os, sys, torch
    sys.path.insert(0, os.environ["FMOE_ROOT"])
    from flash_moe_b200.ops.flash_expert import _expert_forward
    fused = torch.load(os.environ["FMOE_OUT"])
    shapes = [(64, 256, 512, 8), (200, 1024, 2048, 64), (96, 512, 1000, 20), (130, 1000, 777, 70),
              (77, 200, 300, 1), (128, 2048, 4096, 16)]
    worst = 0.0
    for i, (T, H, N, k) in enumerate(shapes):
        g = torch.Generator().manual_seed(100 + i)
        dt = torch.bfloat16
        x = (torch.randn(T, H, generator=g) * 0.5).to(dt).cuda()
        down = (torch.randn(N, H, generator=g) * 0.1).to(dt).cuda()
        up = (torch.randn(N, H, generator=g) * 0.1).to(dt).cuda()
        idx = torch.randint(0, N, (T, k), generator=g).cuda()
        gates = torch.softmax(torch.randn(T, k, generator=g), -1).to(dt).cuda()
        two = _expert_forward(x, down, up, idx, gates, out_dtype=torch.float32).cpu()
        rms = two.pow(2).mean().sqrt()
        worst = max(worst, float((two - fused[i]).abs().max() / rms))
    assert worst < 2e-4, worst  # same float32 sums in another order
    print("two-pass agrees", worst)
    """
)


def _run(script_text, tmp_path, name, env):
    script = tmp_path / name
    script.write_text(script_text)
    res = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


def test_fused_expert_kernel_matches_oracle_and_two_pass(tmp_path):
    out_file = str(tmp_path / "fused_out.pt")
    env = dict(os.environ, FMOE_ROOT=ROOT, FMOE_OUT=out_file, FMOE_EXPERT_SCHEDULE="fused")
    assert "fused cases ok" in _run(WORKER, tmp_path, "fused_worker.py", env)
    env = dict(os.environ, FMOE_ROOT=ROOT, FMOE_OUT=out_file, FMOE_EXPERT_SCHEDULE="token")
    assert "two-pass agrees" in _run(TWO_PASS, tmp_path, "two_pass_worker.py", env)
