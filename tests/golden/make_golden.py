"""Generate the golden fixtures in this directory by running the REFERENCE's own code on CPU.

Needs a checkout of the reference project: pass its path as the first argument or in
``FLASH_MOE_REFERENCE``; it is imported unmodified.  Two sources are used:

* the eager module ``FlashMoE_Pytorch`` (flash_moe/modules/flash_moe.py:108-191),
  with ``cfg.mlp_bias = False`` set on the config object because the class reads
  an attribute ``FlashMoEConfig`` does not define (:122);
* the Triton kernels of the three ops executed by Triton's CPU interpreter
  (``TRITON_INTERPRET=1``), float32 only, with the autotuner pinned to its first
  config (the interpreter cannot benchmark configs).

Run:  python tests/golden/make_golden.py <reference checkout>
Writes ``*.npz`` files next to this script.  The tests only read those files.
"""

import hashlib
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLASH_MOE_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("usage: make_golden.py <path to the flash-moe reference checkout>")
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

import numpy as np  # noqa: E402
import torch  # noqa: E402

from flash_moe.modules.flash_moe import FlashMoE_Pytorch, FlashMoEConfig  # noqa: E402


def params_digest(mod) -> str:
    h = hashlib.sha256()
    for name, p in sorted(mod.state_dict().items()):
        h.update(name.encode())
        h.update(p.detach().float().contiguous().numpy().tobytes())
    return h.hexdigest()


def make_cfg(H, I, N, k, norm):
    cfg = FlashMoEConfig(H, I, "silu", N, k, norm)
    cfg.mlp_bias = False
    return cfg


def eager_routing(mod, x):
    """Re-run the router part of the eager forward to expose scores/indices (flash_moe.py:147-167)."""
    import torch.nn.functional as F

    T = x.shape[0] * x.shape[1]
    logits = mod.router_gate(mod.router_norm(x.view(-1, mod.hidden_size)))
    logits = logits.view(T, 2, -1).transpose(0, 1)
    lp = F.log_softmax(logits, dim=-1)
    (sx, sy), (ix, iy) = lp.topk(mod.num_keys, dim=-1)
    s = (sx.unsqueeze(-1) + sy.unsqueeze(-2)).flatten(-2)
    i = (ix.unsqueeze(-1) * mod.num_keys + iy.unsqueeze(-2)).flatten(-2)
    sc, pos = s.topk(mod.top_k, dim=-1)
    return lp, sc, i.gather(-1, pos)


def layer_case(name, H, I, N, k, norm, B, S, dtype, store_inputs, train=False):
    torch.manual_seed(0)
    mod = FlashMoE_Pytorch(make_cfg(H, I, N, k, norm))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, S, H, generator=g)
    mod = mod.to(dtype)
    x = x.to(dtype)
    mod.train(train)
    digest = params_digest(mod)
    with torch.no_grad():
        # routing first on a copy of the BN buffers so the forward below sees fresh ones
        sd = {k_: v.clone() for k_, v in mod.state_dict().items()}
        lp, sc, idx = eager_routing(mod, x)
        mod.load_state_dict(sd)
        y, logits = mod(x)
    out = {
        "cfg": np.array([H, I, N, k, int(norm), B, S, int(train)], dtype=np.int64),
        "dtype": np.array(str(dtype)),
        "params_sha256": np.array(digest),
        "y": y.float().numpy(),
        "router_logits": logits.contiguous().float().numpy(),
        "log_probs": lp.contiguous().float().numpy(),
        "scores": sc.float().numpy(),
        "indices": idx.numpy(),
        "running_mean_after": mod.router_norm.running_mean.float().numpy(),
        "running_var_after": mod.router_norm.running_var.float().numpy(),
    }
    if store_inputs:
        out["x"] = x.float().numpy()
        for n, p in sd.items():
            out["param." + n] = p.float().numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, "y rms", float(y.float().pow(2).mean().sqrt()), "digest", digest[:12])


def layer_grad_case(name, H, I, N, k, norm, B, S, train=False):
    """Gradients of loss = sum(y * w) through the reference's eager module under torch autograd (float32)."""
    torch.manual_seed(0)
    mod = FlashMoE_Pytorch(make_cfg(H, I, N, k, norm))
    mod.train(train)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, S, H, generator=g, requires_grad=True)
    w = torch.randn(B, S, H, generator=g)
    sd = {k_: v.clone() for k_, v in mod.state_dict().items()}
    y, _ = mod(x)
    (y * w).sum().backward()
    out = {"cfg": np.array([H, I, N, k, int(norm), B, S, int(train)], dtype=np.int64), "x": x.detach().numpy(),
           "w": w.numpy(), "y": y.detach().numpy(), "grad.x": x.grad.numpy()}
    for n, p in mod.named_parameters():
        out["grad." + n] = p.grad.numpy()
    for n, p in sd.items():
        out["param." + n] = p.float().numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, "grad norms", {n: float(p.grad.norm()) for n, p in mod.named_parameters()})


def pin_autotuner(kernel):
    if hasattr(kernel, "configs"):
        kernel.configs = kernel.configs[:1]


def triton_router_case(name, T, nk, k, tied):
    from flash_moe.ops.triton.flash_router import triton_flash_router_func

    g = torch.Generator().manual_seed(7)
    raw = torch.randn(2, T, nk, generator=g)
    if tied:
        raw = torch.round(raw * 2) / 2  # coarse grid -> many exactly equal pair sums
        lp = raw - 4.0
    else:
        lp = torch.log_softmax(raw, dim=-1)
    s, i = triton_flash_router_func(lp, nk, k)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        log_probs=lp.numpy(), nk=np.int64(nk), k=np.int64(k), scores=s.numpy(), indices=i.numpy(),
    )
    print(name, "ok", tuple(i.shape))


def triton_expert_case(name, T, H, N, k):
    import flash_moe.ops.triton.flash_expert as fe

    pin_autotuner(fe._fwd_scores_kernel)
    pin_autotuner(fe._fwd_states_kernel)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g) * 0.5
    d = torch.randn(N, H, generator=g) * 0.1
    u = torch.randn(N, H, generator=g) * 0.1
    idx = torch.randint(0, N, (T, k), generator=g)
    idx[0, 1] = idx[0, 0]  # a duplicated expert inside one token must accumulate
    gates = torch.randn(T, k, generator=g) * 0.1
    y = fe.triton_flash_expert_func(x, d, u, idx, gates)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        x=x.numpy(), down=d.numpy(), up=u.numpy(), indices=idx.numpy(), gates=gates.numpy(), y=y.numpy(),
    )
    print(name, "ok")


def triton_mlp_case(name, T, H, I):
    import flash_moe.ops.triton.flash_mlp as fm

    pin_autotuner(fm._swiglu_forward_kernel)
    g = torch.Generator().manual_seed(13)
    x = torch.randn(T, H, generator=g) * 0.5
    wg = torch.randn(I, H, generator=g) * 0.1
    wu = torch.randn(I, H, generator=g) * 0.1
    wd = torch.randn(H, I, generator=g) * 0.1
    y = fm.triton_flash_mlp_func(x, wg, wu, wd)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x.numpy(), wg=wg.numpy(), wu=wu.numpy(), wd=wd.numpy(), y=y.numpy())
    print(name, "ok")


def triton_peer_pkm_case(name, T, H, N, k):
    import flash_moe.ops.triton.peer as peer
    import flash_moe.ops.triton.pkm as pkm

    pin_autotuner(peer._peer_fwd_kernel)
    pin_autotuner(pkm._pkm_fwd_kernel)
    g = torch.Generator().manual_seed(17)
    x = torch.randn(T, H, generator=g) * 0.5
    d = torch.randn(N, H, generator=g) * 0.3
    u = torch.randn(N, H, generator=g) * 0.3
    idx = torch.randint(0, N, (T, k), generator=g)
    idx[0, 1] = idx[0, 0]
    w = torch.softmax(torch.randn(T, k, generator=g), -1)
    y_peer = peer.triton_peer_func(x, d, u, w, idx)
    y_pkm = pkm.triton_pkm_func(u, w, idx)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x.numpy(), down=d.numpy(), up=u.numpy(), weights=w.numpy(),
                        indices=idx.numpy(), y_peer=y_peer.numpy(), y_pkm=y_pkm.numpy())
    print(name, "ok")


if __name__ == "__main__":
    torch.set_num_threads(os.cpu_count() or 1)
    # eager module: a mini case stored with all inputs, and benchmark configuration 1 stored as outputs + digest
    layer_case("eager_mini_fp32", 64, 128, 256, 4, False, 2, 16, torch.float32, store_inputs=True)
    layer_case("eager_mini_fp32_train_norm", 64, 128, 256, 4, True, 2, 16, torch.float32, store_inputs=True, train=True)
    layer_case("eager_mini_bf16", 64, 128, 256, 4, False, 2, 16, torch.bfloat16, store_inputs=True)
    layer_case("eager_c1_fp32", 256, 1024, 1024, 8, False, 1, 256, torch.float32, store_inputs=False)
    layer_grad_case("eager_mini_fp32_grads", 64, 128, 256, 4, False, 2, 16)
    layer_grad_case("eager_mini_fp32_grads_norm_train", 64, 128, 256, 4, True, 2, 16, train=True)
    # Triton kernels under the interpreter
    triton_router_case("triton_router_nk16_k4", 16, 16, 4, tied=False)
    triton_router_case("triton_router_nk16_k4_tied", 16, 16, 4, tied=True)
    triton_router_case("triton_router_nk32_k8_tied", 8, 32, 8, tied=True)
    triton_router_case("triton_router_nk128_k16", 2, 128, 16, tied=False)
    triton_expert_case("triton_expert_small", 16, 64, 64, 4)
    triton_mlp_case("triton_mlp_small", 8, 32, 64)
    triton_peer_pkm_case("triton_peer_pkm_small", 16, 48, 40, 4)
