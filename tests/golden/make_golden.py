"""Generate the golden fixtures in this folder from the real reference.

Run once, in a container that has the reference checkout (its path is given on
the command line); the resulting ``.npz`` files are committed and are what the
tests read.  Nothing else in the repository imports the reference.

    python tests/golden/make_golden.py <path-to-reference-checkout>

Each fixture stores the construction recipe (d, r, L, seed, alpha, jitter), the
bf16 input rows as raw uint16 bits, and the reference module's outputs:
``y_bf16`` (module in bf16, raw bits) and ``y_fp32`` (module in fp32 loaded with
the bf16-rounded weights and input).  Parameters are not stored: they are a
pure function of the seed (dlr_lock/model.py:65-81 draw order), and two short
checksums pin that the oracle's generator reproduces them.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def build_case(DLRNet, d, r, L, M, seed, alpha, jitter):
    torch.manual_seed(seed)
    net = DLRNet(d, r, L, alpha_init=alpha)          # draws V then U
    if jitter:
        with torch.no_grad():
            for w in net.rms_w:
                w.add_(jitter * torch.randn(d))
    x = torch.randn(M, d)
    net_bf = DLRNet(d, r, L, alpha_init=alpha)
    net_bf.load_state_dict(net.state_dict())
    net_bf = net_bf.to(torch.bfloat16)
    xb = x.to(torch.bfloat16)
    net32 = DLRNet(d, r, L, alpha_init=alpha)
    net32.load_state_dict({k: v.float() for k, v in net_bf.state_dict().items()})
    with torch.no_grad():
        y_bf = net_bf(xb)
        y_32 = net32(xb.float())
    v_sum = float(sum(v.double().sum() for v in net.Vs))
    u_sum = float(sum(u.double().sum() for u in net.Us))
    return net_bf, xb, y_bf, y_32, v_sum, u_sum


def write_bench_twin(kref):
    """Checksums of the benchmark twin of the net (kernels/reference.py:46-55: U drawn before V, alpha 0.01)
    built as kernels/reference.py:94-102 does (seed 42), on the CPU, and its packed weights' checksums."""
    out = {}
    for name in ("Qwen3-0.6B",):
        cfg = kref.MODEL_CONFIGS[name]
        depth = kref.compute_depth(cfg["d"], cfg["d_ff"], cfg["r"])
        torch.manual_seed(42)
        net = kref.DLRNet(cfg["d"], cfg["r"], depth).to(kref.DTYPE)
        packed = kref.pack_dlrnet_weights(net, device="cpu", premultiply=True)
        out[name] = dict(depth=depth,
                         u_sum=float(sum(u.double().sum() for u in net.Us)), v_sum=float(sum(v.double().sum() for v in net.Vs)),
                         u0_first=float(net.Us[0].flatten()[0]), v0_first=float(net.Vs[0].flatten()[0]),
                         alpha=float(net.alphas[0]),
                         packed_Vs_sum=float(packed["Vs"].double().sum()), packed_Us_sum=float(packed["Us"].double().sum()),
                         packed_Vs_shape=list(packed["Vs"].shape), packed_Us_shape=list(packed["Us"].shape))
    with open(os.path.join(HERE, "bench_twin.json"), "w") as f:
        json.dump(out, f, indent=1)


def main():
    ref = sys.argv[1]
    sys.path.insert(0, ref)
    sys.path.insert(0, os.path.join(ref, "kernels"))
    from dlr_lock.model import DLRNet, compute_depth, dlrnet_param_count
    import reference as kref

    write_bench_twin(kref)
    if "--twin-only" in sys.argv:
        return

    torch.set_num_threads(8)
    cases = [
        # name, d, r, L, M, seed, alpha, gain jitter
        ("toy_d64_r8", 64, 8, 12, 28, 7, 0.1, 0.0),            # smoke-test shape
        ("toy_d256_r32", 256, 32, 5, 9, 11, 0.01, 0.0),
        ("toy_d256_r32_stress", 256, 32, 24, 9, 12, 1.0, 0.1),
        ("toy_d512_r64_stress", 512, 64, 17, 70, 13, 1.0, 0.1),
        ("cfg1_d1024_r32", 1024, 32, 141, 16, 0, 0.01, 0.0),
        ("cfg1_d1024_r32_stress", 1024, 32, 141, 16, 100, 1.0, 0.1),
        ("cfg2_d2048_r64", 2048, 64, 142, 4, 1, 0.01, 0.0),
        ("cfg3_d4096_r128", 4096, 128, 143, 4, 2, 0.01, 0.0),
        ("cfg4_d5120_r256", 5120, 256, 149, 2, 3, 0.01, 0.0),
    ]
    for name, d, r, L, M, seed, alpha, jitter in cases:
        net_bf, xb, y_bf, y_32, v_sum, u_sum = build_case(DLRNet, d, r, L, M, seed, alpha, jitter)
        out = dict(
            meta=json.dumps(dict(d=d, r=r, L=L, M=M, seed=seed, alpha=alpha,
                                 gain_jitter=jitter, v_sum=v_sum, u_sum=u_sum)),
            x_bits=bits(xb), y_bf16_bits=bits(y_bf), y_fp32=y_32.numpy(),
        )
        if d <= 256:
            # folded weights of the reference packer (kernels/reference.py:68-91):
            # Vs is (L,D,R) = V'^T, Us is (L,R,D) = U'^T.
            packed = kref.pack_dlrnet_weights(net_bf, device="cpu", premultiply=True)
            out["packed_Vs_bits"] = bits(packed["Vs"])
            out["packed_Us_bits"] = bits(packed["Us"])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "written")

    table = {f"{d},{d_ff},{r}": [compute_depth(d, d_ff, r), dlrnet_param_count(d, r, compute_depth(d, d_ff, r))]
             for d, d_ff, r in ((1024, 3072, 32), (2048, 6144, 64), (4096, 12288, 128),
                                (5120, 25600, 256), (64, 256, 8), (1024, 3072, 16))}
    with open(os.path.join(HERE, "depth_table.json"), "w") as f:
        json.dump(table, f, indent=1)


if __name__ == "__main__":
    main()
