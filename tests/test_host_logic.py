"""Host-side mirror of the reference API, on CPU."""
import os

import pytest
import torch

import dlr_lock_b200 as D
from dlr_lock_b200 import registry, sharding
from oracle import dlrnet_oracle as O

from conftest import load_golden


def test_module_matches_oracle_and_reference_fixture():
    g = load_golden("toy_d256_r32_stress")
    m = g["meta"]
    p = O.seeded_params(m["d"], m["r"], m["L"], m["seed"], m["alpha"], m["gain_jitter"]).to(torch.bfloat16)
    net = D.DLRNet(m["d"], m["r"], m["L"], alpha_init=m["alpha"])
    sd = {}
    for i in range(m["L"]):
        sd[f"Vs.{i}"], sd[f"Us.{i}"], sd[f"rms_w.{i}"], sd[f"alphas.{i}"] = p.V[i], p.U[i], p.w[i], p.alpha[i]
    net.load_state_dict(sd)                      # reference state_dict keys (dlr_lock/model.py:232-248)
    net = net.to(torch.bfloat16)
    with torch.no_grad():
        y = net(g["x"])
    assert O.rel_l2(y, g["y_bf16"]) <= 2e-3


def test_invariants_of_the_reference_smoke_test():
    # examples/smoke_test.py:65-98
    d, r, depth = 64, 8, 12
    net = D.DLRNet(d, r, depth, alpha_init=0.0)
    assert sum(p.numel() for p in net.parameters()) == D.dlrnet_param_count(d, r, depth)
    x = torch.randn(4, 7, d)
    assert torch.equal(net(x), x)
    net = D.DLRNet(d, r, depth, alpha_init=0.1)
    xg = torch.randn(3, 5, d, requires_grad=True)
    net.use_checkpoint = True
    ya = net(xg)
    ga = torch.autograd.grad(ya.sum(), xg)[0]
    net.use_checkpoint = False
    yb = net(xg)
    gb = torch.autograd.grad(yb.sum(), xg)[0]
    assert torch.allclose(ya, yb, atol=1e-6) and torch.allclose(ga, gb, atol=1e-6)
    for dd, d_ff, rr, want in ((1024, 3072, 32, 141), (2048, 6144, 64, 142), (4096, 12288, 128, 143),
                               (5120, 25600, 256, 149)):
        assert D.compute_depth(dd, d_ff, rr) == want
    cfg = D.dlrnet_config(1024, 3072, 32)
    assert cfg["depth"] == 141 and cfg["params"] == D.dlrnet_param_count(1024, 32, 141)


def test_cuda_only_entry_points_refuse_cpu_tensors():
    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    V = torch.zeros(3, 16, 64, dtype=torch.bfloat16)
    U = torch.zeros(3, 64, 16, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        D.ops.forward_folded(x, V, U)
    with pytest.raises(ValueError):
        D.ops.fold_weights(V, U, torch.ones(3, 64), torch.ones(3))


def test_registry_covers_every_cell():
    for model in ("Qwen3-0.6B", "Qwen3-1.7B", "Qwen3-8B", "Qwen3-32B"):
        for B in (1, 2, 8, 64, 65, 1024, 6000, 8192, 131072):
            e = registry.resolve(model, B)
            assert e is not None and set(e) >= {"B_lo", "B_hi", "kernel", "callable", "config", "note"}
            mod, fn = e["callable"].rsplit(".", 1)
            assert callable(getattr(__import__(mod, fromlist=[fn]), fn))
    assert registry.resolve("Qwen3-8B", 0) is None
    assert registry.resolve("nope", 4) is None


@pytest.mark.parametrize("M,world,tile", [(8192, 8, 128), (1000, 4, 128), (3, 8, 1), (0, 2, 16), (129, 2, 128)])
def test_row_blocks_partition(M, world, tile):
    blocks = sharding.row_blocks(M, world, tile)
    assert len(blocks) == world and blocks[0][0] == 0 and blocks[-1][1] == M
    for (a, b), (c, _) in zip(blocks, blocks[1:]):
        assert a <= b == c
    for a, b in blocks[:-1]:
        assert (b - a) % tile == 0 or b == M


def _tiny_qwen3(tmp_path):
    from transformers import AutoConfig, AutoModelForCausalLM
    cfg = AutoConfig.for_model("qwen3", vocab_size=128, hidden_size=64, intermediate_size=256,
                               num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                               head_dim=16, max_position_embeddings=64, tie_word_embeddings=True)
    path = os.path.join(tmp_path, "tiny")
    AutoModelForCausalLM.from_config(cfg).save_pretrained(path)
    return path


def test_surgery_and_checkpoint_round_trip(tmp_path):
    # examples/smoke_test.py:101-124 and 156-188, on a random two-layer decoder
    path = _tiny_qwen3(str(tmp_path))
    torch.manual_seed(0)
    model = D.build_locked_model(path, rank=8, torch_dtype=torch.float32, alpha_init=0.1, verbose=False).eval()
    depth = D.compute_depth(64, 256, 8)
    assert model.model.layers[0].mlp.dlrnet.depth == depth
    seen = {}
    layer = model.model.layers[1]
    h1 = layer.mlp.register_forward_hook(lambda m, a, o: seen.__setitem__("h", a[0].detach()))
    h2 = layer.register_forward_hook(lambda m, a, o: seen.__setitem__("out", (o[0] if isinstance(o, tuple) else o).detach()))
    ids = torch.randint(0, 128, (2, 9))
    with torch.no_grad():
        logits = model(ids).logits
    h1.remove(); h2.remove()
    with torch.no_grad():
        want = layer.mlp.dlrnet(seen["h"])
    assert torch.allclose(seen["out"], want, atol=1e-5)

    ckpt = os.path.join(str(tmp_path), "ckpt")
    assert D.save_dlrnet_weights(model, ckpt) == 2
    assert sorted(os.listdir(ckpt)) == ["layer00.pt", "layer01.pt"]
    sd = torch.load(os.path.join(ckpt, "layer00.pt"), weights_only=True)
    assert {"Vs.0", "Us.0", "rms_w.0", "alphas.0"} <= set(sd)
    fresh = D.build_locked_model(path, rank=8, torch_dtype=torch.float32, alpha_init=0.0, verbose=False).eval()
    assert D.load_dlrnet_weights(fresh, ckpt) == 2
    with torch.no_grad():
        again = fresh(ids).logits
    assert torch.allclose(logits, again, atol=1e-6)
    assert D.set_checkpointing(fresh, False) == 2
    assert D.accelerate_locked_model(fresh) == 2


def test_fast_path_is_refused_whenever_a_gradient_could_be_asked_for():
    # eval mode + grad enabled + trainable parameters: the library's output would be detached from the
    # parameters, so the module must take the torch loop (dlr_lock/model.py:88-101 always builds the graph)
    net = D.DLRNet(64, 8, 3, alpha_init=0.1).to(torch.bfloat16).eval()
    x = torch.randn(2, 64, dtype=torch.bfloat16)

    class X:      # what _fast_ok looks at, standing in for a CUDA bf16 input on a machine without a GPU
        is_cuda, dtype, requires_grad = True, torch.bfloat16, False
    with torch.enable_grad():
        assert net._fast_ok(X) is False                    # parameters require grad, eval mode
        net.Vs[0].requires_grad_(False)
        assert net._fast_ok(X) is False                    # first V frozen, the others still train
        for p in net.parameters():
            p.requires_grad_(False)
        assert net._fast_ok(X) is True
        X.requires_grad = True
        assert net._fast_ok(X) is False
    with torch.no_grad():
        for p in net.parameters():
            p.requires_grad_(True)
        X.requires_grad = False
        assert net._fast_ok(X) is True                     # inference: nothing can ask for a gradient
    # and the torch loop it falls back to does carry gradients to a middle layer's parameters
    net.train()
    net(x).float().sum().backward()
    assert net.Us[1].grad is not None


def test_folded_cache_key_sees_an_edit_of_any_layer():
    net = D.DLRNet(64, 8, 5, alpha_init=0.1)
    k0 = net._cache_key()
    with torch.no_grad():
        net.rms_w[2].mul_(1.5)                             # in-place edit of a middle layer
    k1 = net._cache_key()
    assert k1 != k0
    with torch.no_grad():
        net.alphas[3].fill_(0.3)
    assert net._cache_key() != k1
    k2 = net._cache_key()
    net.Vs[1].data.copy_(torch.zeros_like(net.Vs[1]))      # bypasses the version counter: documented, needs invalidate()
    assert net._cache_key() == k2
    net._folded = ("sentinel",)
    net.invalidate()
    assert net._folded is None


def test_fused_decoder_layer_equals_the_reference_composition(tmp_path):
    # dlr_lock/model.py:121-122 returns dlrnet(h) - h and the host layer adds h back; the fused layer
    # forward returns dlrnet(h) directly.  In fp32 on the CPU the two agree to rounding.
    path = _tiny_qwen3(str(tmp_path))
    model = D.build_locked_model(path, rank=8, torch_dtype=torch.float32, alpha_init=0.3, verbose=False).eval()
    ids = torch.randint(0, 128, (2, 7))
    with torch.no_grad():
        want = model(ids).logits
        assert D.fuse_decoder_layers(model, True) == len(model.model.layers)
        got = model(ids).logits
        out = model(ids[:, :5], use_cache=True)                       # the KV cache path goes through the same forward
        step = model(ids[:, 5:6], past_key_values=out.past_key_values, use_cache=True).logits
        assert D.fuse_decoder_layers(model, False) == len(model.model.layers)
        back = model(ids).logits
        ref_step = model(ids[:, :6]).logits[:, -1:]
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
    assert torch.equal(back, want)
    assert torch.allclose(step, ref_step, atol=1e-4, rtol=1e-4)


def test_perplexity_consumer_on_cpu(tmp_path):
    # dlr_lock/eval_benchmarks.py:89-100 on the synthetic stream: deterministic, finite, and equal for the same seed
    path = _tiny_qwen3(str(tmp_path))
    model = D.build_locked_model(path, rank=8, torch_dtype=torch.float32, alpha_init=0.1, verbose=False).eval()
    a = D.evaluate_ppl(model, D.synthetic_token_stream(128, 16, 2, seed=7), n_steps=3, device="cpu")
    b = D.evaluate_ppl(model, D.synthetic_token_stream(128, 16, 2, seed=7), n_steps=3, device="cpu")
    assert a == b and 1.0 < a < 1e4
    s = D.synthetic_token_stream(128, 16, 2, seed=7)
    x = next(s)
    assert x.shape == (2, 16) and x.dtype == torch.long and int(x.max()) < 128
    with pytest.raises(ValueError):
        D.synthetic_token_stream(128, 100000, 2)


def test_bench_harness_twin_packer_and_cell_gate():
    # the benchmark twin and packer against checksums written from the reference's own kernels/reference.py
    # (tests/golden/bench_twin.json), and the ok / WRONG gate of the cell harness on the CPU
    import json
    import os
    from conftest import GOLDEN
    from dlr_lock_b200 import harness
    with open(os.path.join(GOLDEN, "bench_twin.json")) as f:
        want = json.load(f)["Qwen3-0.6B"]
    swiglu, net, cfg = harness.build_models("Qwen3-0.6B", seed=42, device="cpu")
    assert cfg["depth"] == want["depth"] == 141 and abs(float(net.alphas[0]) - want["alpha"]) < 1e-3
    assert abs(float(sum(u.double().sum() for u in net.Us)) - want["u_sum"]) < 1e-6
    assert abs(float(sum(v.double().sum() for v in net.Vs)) - want["v_sum"]) < 1e-6
    assert float(net.Us[0].flatten()[0]) == want["u0_first"] and float(net.Vs[0].flatten()[0]) == want["v0_first"]
    packed = harness.pack_dlrnet_weights(net, premultiply=True)
    assert list(packed["Vs"].shape) == want["packed_Vs_shape"] and list(packed["Us"].shape) == want["packed_Us_shape"]
    assert abs(float(packed["Vs"].double().sum()) - want["packed_Vs_sum"]) < 1e-9
    assert abs(float(packed["Us"].double().sum()) - want["packed_Us_sum"]) < 1e-9
    assert packed["premultiplied"] and packed["L"] == 141 and packed["D"] == 1024 and packed["R"] == 32
    assert swiglu.gate_proj.weight.shape == (3072, 1024)
    # gate: an identity "kernel" passes the total-error gate of the reference's harness and is exposed by the
    # update error; a kernel that returns noise is WRONG
    x = torch.randn(4, 1024).to(torch.bfloat16)
    with torch.no_grad():
        ref = net._forward_impl(x)
    assert harness.rel_err(x, ref) <= harness.REL_ERR_TOL and harness.update_err(x, ref, x) > 0.99
    assert harness.update_err(ref, ref, x) == 0.0
