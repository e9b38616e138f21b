"""The locked decoder loop end to end: a randomly initialised Qwen3-shaped decoder whose MLPs are
DLR-Nets (28 layers, hidden 1024, 16 query / 8 key-value heads of 128, rank 32, depth 141), run once
through the CUDA library and once through the torch layer loop (dlr_lock/model.py:93-101 restated in
dlr_lock_b200.model.DLRNet._forward_impl), the way examples/smoke_test.py:101-124 compares surgery
results.  Logits are compared under teacher forcing: the prefill, then single-token steps fed with the
torch path's greedy tokens, each path on its own KV cache.  Sampled ids of a random model are not
compared: an argmax tie flips on a one-ulp difference.
"""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


def test_locked_decoder_prefill_and_decode_logits():
    import dlr_lock_b200 as D
    from transformers import AutoConfig

    dev = "cuda:0"
    torch.manual_seed(0)
    cfg = AutoConfig.for_model("qwen3", vocab_size=8192, hidden_size=1024, intermediate_size=3072,
                               num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                               max_position_embeddings=2048, tie_word_embeddings=True)
    model = D.locked_model_from_config(cfg, rank=32, device=dev, alpha_init=0.01).eval()
    assert D.set_fast_path(model, True) == 28
    assert model.model.layers[0].mlp.dlrnet.depth == D.compute_depth(1024, 3072, 32) == 141
    truth = copy.deepcopy(model).float()          # same bf16-rounded weights, everything computed in fp32
    D.set_fast_path(truth, False)

    ids = torch.randint(0, 8192, (2, 48), device=dev)
    with torch.no_grad():
        D.set_fast_path(model, False)
        eager = model(ids, use_cache=True)
        D.set_fast_path(model, True)
        fast = model(ids, use_cache=True)
        want = truth(ids, use_cache=True)
        torch.cuda.synchronize()
        D.ops.check_status()
        # the library against the torch loop in bf16, and both against the fp32 model: the library must not
        # be further from the truth than the reference arithmetic is
        assert _rel(fast.logits, eager.logits) <= 3e-2
        e_fast, e_eager = _rel(fast.logits, want.logits), _rel(eager.logits, want.logits)
        assert e_fast <= 1.25 * e_eager + 2e-3, (e_fast, e_eager)
        # near-ties of a random model flip on one ulp: most positions agree, not all
        assert (fast.logits.argmax(-1) == eager.logits.argmax(-1)).float().mean().item() >= 0.85
        # the fused layer forward (attention output straight into the net, the net's output as the layer's
        # output, dlr_lock/model.py:121-122's "- h" and the host layer's "+ h" never run): same gates, and no
        # further from the fp32 model than the reference composition
        assert D.fuse_decoder_layers(model, True) == 28
        fused = model(ids, use_cache=True)
        torch.cuda.synchronize()
        D.ops.check_status()
        assert _rel(fused.logits, eager.logits) <= 3e-2
        assert _rel(fused.logits, want.logits) <= 1.25 * e_eager + 2e-3
        pu = fused.past_key_values

        pe, pf = eager.past_key_values, fast.past_key_values
        tok = eager.logits[:, -1:].argmax(-1)
        for _ in range(3):
            D.fuse_decoder_layers(model, False)
            D.set_fast_path(model, False)
            oe = model(tok, past_key_values=pe, use_cache=True)
            pe = oe.past_key_values
            D.set_fast_path(model, True)
            D.fuse_decoder_layers(model, False)
            of = model(tok, past_key_values=pf, use_cache=True)
            pf = of.past_key_values
            D.fuse_decoder_layers(model, True)
            ou = model(tok, past_key_values=pu, use_cache=True)
            pu = ou.past_key_values
            torch.cuda.synchronize()
            D.ops.check_status()
            assert _rel(of.logits, oe.logits) <= 3e-2
            assert _rel(ou.logits, oe.logits) <= 3e-2
            tok = oe.logits[:, -1:].argmax(-1)


def test_perplexity_with_the_library_matches_the_torch_loop():
    # dlr_lock/eval_benchmarks.py:89-100 on a synthetic token stream (the stand-in of examples/smoke_test.py:40-48
    # for the corpus): the locked model's perplexity with the CUDA library under its nets, with the fused layer
    # forward on top, and with the torch layer loop agree within one percent
    import dlr_lock_b200 as D
    from transformers import AutoConfig

    dev = "cuda:0"
    torch.manual_seed(3)
    cfg = AutoConfig.for_model("qwen3", vocab_size=4096, hidden_size=1024, intermediate_size=3072,
                               num_hidden_layers=8, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                               max_position_embeddings=2048, tie_word_embeddings=True)
    model = D.locked_model_from_config(cfg, rank=32, device=dev, alpha_init=0.01).eval()
    ppl = {}
    for name, fast, fused in (("torch_loop", False, False), ("library", True, False), ("library_fused", True, True)):
        D.set_fast_path(model, fast)
        D.fuse_decoder_layers(model, fused)
        ppl[name] = D.evaluate_ppl(model, D.synthetic_token_stream(4096, 256, 4, seed=42), n_steps=4, device=dev)
    torch.cuda.synchronize()
    D.ops.check_status()
    assert all(v == v and v > 1.0 for v in ppl.values()), ppl           # finite, and a loss was computed
    assert abs(ppl["library"] / ppl["torch_loop"] - 1.0) <= 1e-2, ppl
    assert abs(ppl["library_fused"] / ppl["torch_loop"] - 1.0) <= 1e-2, ppl


def test_checkpoint_to_packed_weights(tmp_path):
    # layerNN.pt files written by save_dlrnet_weights, read straight into folded device stacks: the same
    # bits as the module computes from the same parameters, with and without the packed cache
    import os

    import dlr_lock_b200 as D
    from transformers import AutoConfig

    dev = "cuda:0"
    torch.manual_seed(1)
    cfg = AutoConfig.for_model("qwen3", vocab_size=128, hidden_size=512, intermediate_size=1536, num_hidden_layers=2,
                               num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=64,
                               tie_word_embeddings=True)
    model = D.locked_model_from_config(cfg, rank=64, device=dev, alpha_init=0.3).eval()
    ckpt = str(tmp_path / "ckpt")
    assert D.save_dlrnet_weights(model, ckpt) == 2
    x = torch.randn(70, 512, device=dev).to(torch.bfloat16)
    with torch.no_grad():
        want = [layer.mlp.dlrnet(x) for layer in model.model.layers]
    nets = D.load_packed_weights(ckpt, dev, write_cache=True)
    assert len(nets) == 2 and nets[0].d == 512 and nets[0].r == 64 and nets[0].depth == model.model.layers[0].mlp.dlrnet.depth
    assert sorted(os.listdir(os.path.join(ckpt, "packed_b200"))) == ["layer00.pt", "layer01.pt"]
    again = D.load_packed_weights(ckpt, dev)                       # served from the packed cache
    torch.cuda.synchronize()
    for w, a, b in zip(want, nets, again):
        assert torch.equal(a(x), w) and torch.equal(b(x), w)
    D.ops.check_status()
    with pytest.raises(ValueError):
        D.pack_state_dict({"Vs.0": torch.zeros(4, 8)}, dev)
    # an fp32 checkpoint, as the reference's distillation writes it (dlr_lock/distill_logits.py:196-200): the
    # serving module holds it in bf16 (alpha included) before folding, and so does the packed path
    net32 = D.DLRNet(512, 64, 5, alpha_init=0.0123456)
    with torch.no_grad():
        for w in net32.rms_w:
            w.add_(0.1 * torch.randn(512))
    ckpt32 = str(tmp_path / "ckpt32")
    os.makedirs(ckpt32)
    torch.save(net32.state_dict(), os.path.join(ckpt32, "layer00.pt"))
    served = D.DLRNet(512, 64, 5)
    served.load_state_dict(torch.load(os.path.join(ckpt32, "layer00.pt"), weights_only=True))
    served = served.to(dev).to(torch.bfloat16).eval()
    (packed32,) = D.load_packed_weights(ckpt32, dev, n_layers=1, eps=1e-6)
    Vp, Up = served.folded_weights()
    assert torch.equal(packed32.Vp, Vp) and torch.equal(packed32.Up, Up)
    # the caller's epsilon applies on a cache hit, not the one stored with the packed stacks
    D.load_packed_weights(ckpt32, dev, n_layers=1, eps=1e-6, write_cache=True)
    (hit,) = D.load_packed_weights(ckpt32, dev, n_layers=1, eps=1e-5)
    assert hit.eps == 1e-5 and torch.equal(hit.Vp, Vp)
