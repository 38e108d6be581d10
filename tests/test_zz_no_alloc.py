"""`fmoe_expert_forward_static`: the expert forward for hosts that cannot give the library scratch
memory (frozen memory plans, fixed real-time budgets, bindings without a device allocator).

The test drives the C ABI directly with ctypes - no workspace tensor is created for the new entry
point - and compares it with `fmoe_expert_forward` on the same inputs, twice in a row because the
built-in scratch array keeps the previous call's contents.  It lives in a file of its own that
pytest collects last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(T, H, N, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) * 0.5).to(dtype).cuda()
    d = (torch.randn(N, H, generator=g) * 0.1).to(dtype).cuda()
    u = (torch.randn(N, H, generator=g) * 0.1).to(dtype).cuda()
    idx = torch.randint(0, N, (T, k), generator=g).cuda()
    gates = torch.softmax(torch.randn(T, k, generator=g), -1).to(dtype).cuda()
    return x, d, u, idx, gates


def _call(fn_name, tensors, T, H, N, k, dtype, with_workspace):
    from flash_moe_b200 import _lib

    L = _lib.lib()
    x, d, u, idx, gates = tensors
    out = torch.empty(T, H, dtype=torch.float32, device="cuda")
    code = _lib.DTYPE_CODE[dtype]
    stream = torch.cuda.current_stream().cuda_stream
    status = _lib.status_word(x.device).data_ptr()
    args = [x.data_ptr(), d.data_ptr(), u.data_ptr(), idx.data_ptr(), gates.data_ptr(), out.data_ptr(), code, 0, T, H, N, k]
    if with_workspace:
        nbytes = L.fmoe_expert_workspace_bytes(T, H, N, k)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        args += [ws.data_ptr(), nbytes]
    rc = getattr(L, fn_name)(*args, status, stream)
    torch.cuda.synchronize()
    return rc, out


# the first shape takes the gather-per-token schedule, the second (float32) the expert-centric
# sort whose counters live in the scratch and must be re-zeroed by every call
@pytest.mark.parametrize("T,H,N,k,dtype", [(256, 512, 2048, 16, torch.bfloat16), (192, 256, 4096, 8, torch.float32)])
def test_static_scratch_entry_point_matches_workspace_entry_point(T, H, N, k, dtype):
    from flash_moe_b200 import _lib

    L = _lib.lib()
    assert L.fmoe_expert_workspace_bytes(T, H, N, k) <= L.fmoe_expert_static_scratch_bytes()
    for round_ in range(2):
        tensors = _inputs(T, H, N, k, dtype, seed=round_)
        rc_ref, want = _call("fmoe_expert_forward", tensors, T, H, N, k, dtype, with_workspace=True)
        rc_new, got = _call("fmoe_expert_forward_static", tensors, T, H, N, k, dtype, with_workspace=False)
        assert rc_ref == 0 and rc_new == 0
        # same kernels, same order of accumulation: the tolerance of the other expert tests (2e-5 x 10
        # of RMS for the fp32 accumulator) is met with room to spare - the results are bit-equal
        rms = want.double().pow(2).mean().sqrt().item()
        assert (got.double() - want.double()).abs().max().item() <= 2e-4 * rms
        assert torch.equal(got, want)
    assert _lib.read_status() == 0


def test_static_scratch_rejects_shapes_beyond_its_size():
    from flash_moe_b200 import _lib

    L = _lib.lib()
    T, H, N, k = 32768, 256, 1 << 20, 16  # needs far more than the built-in 8 MiB
    assert L.fmoe_expert_workspace_bytes(T, H, N, k) > L.fmoe_expert_static_scratch_bytes()
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    rc = L.fmoe_expert_forward_static(one, one, one, one, one, one, 1, 0, T, H, N, k, None, None)
    assert rc == 3  # FMOE_ERR_WORKSPACE
    assert b"workspace" in L.fmoe_error_string(rc)
