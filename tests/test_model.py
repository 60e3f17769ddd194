"""Model semantics on CPU fp32 (the oracle): shapes, gradients, state-dict names, MoE capacity, MoD skipping, KV cache."""
import math

import pytest
import torch

from adaptivetrainingsystem_b200 import ops
from adaptivetrainingsystem_b200.config import ConfigPresets, ModelConfig
from adaptivetrainingsystem_b200.models import (DeepSeekTransformer, GroupedQueryAttention, MoDFFN, MoEFFNLayer, RMSNorm,
                                                RotaryEmbedding, SwiGLUExpert)
from adaptivetrainingsystem_b200.ops import moe as M

BASE = dict(vocab_size=1000, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=256, seq_length=64)


def test_rmsnorm_shape_and_extreme_inputs():
    n = RMSNorm(128)
    for scale in (1.0, 1e6, 1e-6):
        y = n(torch.randn(2, 16, 128) * scale)
        assert y.shape == (2, 16, 128) and torch.isfinite(y).all()
    x = torch.randn(4, 128)
    assert torch.allclose(n(x).pow(2).mean(-1), torch.ones(4), atol=1e-3)


def test_rope_cache_extends_and_rotation_preserves_norm():
    r = RotaryEmbedding(32, 16)
    cos, sin = r(16)
    assert cos.shape == (16, 16)
    cos, sin = r(100)
    assert cos.shape == (100, 16) and r.cos.shape[0] >= 100
    x = torch.randn(1, 100, 2, 32)
    y = ops.rope_reference(x, r.cos, r.sin, torch.arange(100))
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-4)
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)  # position 0 is the identity


def test_attention_is_causal_and_respects_padding_mask():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 8, 4, 16), torch.randn(1, 8, 2, 16), torch.randn(1, 8, 2, 16)
    o1 = ops.attention_reference(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[:, 5:], v2[:, 5:] = 9.0, 9.0  # the future must not matter
    o2 = ops.attention_reference(q, k2, v2)
    assert torch.allclose(o1[:, :5], o2[:, :5], atol=1e-6)
    mask = torch.ones(1, 8)
    mask[:, 0] = 0
    o3 = ops.attention_reference(q, k, v, key_mask=mask)
    assert torch.isfinite(o3).all() and not torch.allclose(o3[:, 3], o1[:, 3])


def test_expert_and_moe_layer():
    e = SwiGLUExpert(128, 256)
    assert e(torch.randn(5, 128)).shape == (5, 128)
    cfg = ModelConfig(**BASE, use_moe=True, num_experts=4, moe_top_k=2)
    layer = MoEFFNLayer(cfg, 0)
    for p in layer.parameters():
        torch.nn.init.normal_(p, std=0.02)
    out, aux = layer(torch.randn(2, 16, 128))
    assert out.shape == (2, 16, 128) and aux.item() >= 0
    st = layer.get_routing_stats()
    assert abs(sum(st["expert_usage"]) - 1.0) < 1e-6


def test_full_forward_backward_every_parameter_gets_a_gradient():
    for kw in (dict(), dict(use_moe=True, num_experts=4), dict(use_mod=True), dict(use_moe=True, num_experts=4, use_mod=True, moe_pattern="every_2nd")):
        torch.manual_seed(0)
        m = DeepSeekTransformer(ModelConfig(**BASE, tie_word_embeddings=False, **kw))
        ids = torch.randint(0, 1000, (2, 32))
        out = m(ids)
        logits = out[0] if isinstance(out, tuple) else out
        assert logits.shape == (2, 32, 1000)
        res = m.forward_loss(ids, torch.roll(ids, -1, 1))
        res["loss"].backward()
        missing = [n for n, p in m.named_parameters() if p.grad is None]
        assert not missing, (kw, missing)
        assert abs(res["lm_loss"].item() - math.log(1000)) < 0.5


def test_state_dict_uses_reference_names_and_round_trips():
    cfg = ModelConfig(**BASE, use_moe=True, num_experts=4, moe_pattern="odd", use_mod=True)
    m = DeepSeekTransformer(cfg)
    sd = m.state_dict()
    for k in ("embed_tokens.weight", "layers.0.input_norm.weight", "layers.0.self_attn.q_proj.weight", "layers.0.self_attn.k_proj.weight",
              "layers.0.self_attn.v_proj.weight", "layers.0.self_attn.o_proj.weight", "layers.0.post_attn_norm.weight",
              "layers.0.ffn.gate_up_proj.weight", "layers.0.ffn.down_proj.weight", "layers.0.ffn.router.router.weight",
              "layers.0.ffn.router.router.bias", "layers.1.ffn.gate.weight", "layers.1.ffn.experts.3.gate_up_proj.weight",
              "layers.1.ffn.experts.0.down_proj.weight", "norm.weight", "lm_head.weight"):
        assert k in sd, k
    assert sd["layers.0.self_attn.k_proj.weight"].shape == (2 * 32, 128)
    assert sd["layers.0.ffn.gate_up_proj.weight"].shape == (512, 128)
    m2 = DeepSeekTransformer(cfg)
    m2.load_state_dict(sd)
    ids = torch.randint(0, 1000, (1, 16))
    assert torch.equal(m(ids)[0], m2(ids)[0])


def test_capacity_drops_tokens_in_order():
    idx = torch.zeros(10, 1, dtype=torch.int32)  # everyone wants expert 0
    pos, counts, totals = M.plan_slots(idx, 4, 4)
    assert pos.tolist() == [0, 1, 2, 3] + [-1] * 6 and counts.tolist() == [4, 0, 0, 0] and totals.tolist() == [10, 0, 0, 0]
    torch.manual_seed(0)
    x = torch.randn(10, 8)
    w1, w2 = torch.randn(4, 16, 8) * 0.1, torch.randn(4, 8, 8) * 0.1
    out, _ = M.moe_ffn(x, idx, torch.ones(10, 1), w1, w2, 4)
    assert out[4:].abs().max() == 0 and out[:4].abs().max() > 0
    ref = M.moe_ffn_reference(x, idx, torch.ones(10, 1), w1, w2, 4)
    assert torch.allclose(out, ref, atol=1e-5)


def test_dropless_routing_is_selectable_from_config_and_matches_the_per_expert_loop():
    """Skewed routing: one expert is wanted by every token, far more than capacity_factor allows.  ``Config(drop_tokens=False)``
    reaches the layer and gives the dropless result of the reference's live MoE layer (every routed token is computed);
    the default enforces the capacity and matches the oracle with that capacity."""
    from adaptivetrainingsystem_b200.config import Config
    T, E, k = 512, 4, 2
    x = torch.rand(T, 32, generator=torch.Generator().manual_seed(1)) + 0.1
    outs = {}
    for drop in (False, True):
        cfg = Config(vocab_size=256, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=48, seq_length=64,
                     use_moe=True, num_experts=E, moe_top_k=k, capacity_factor=1.25, drop_tokens=drop, precision="fp32",
                     gradient_checkpointing=False)
        mc = cfg.to_model_config()
        assert mc.drop_tokens is drop
        torch.manual_seed(3)
        layer = MoEFFNLayer(mc, 0).train()  # training mode keeps the routing statistics (routing noise is off in this config)
        with torch.no_grad():
            torch.nn.init.normal_(layer.experts_w1, std=0.1)
            torch.nn.init.normal_(layer.experts_w2, std=0.1)
            layer.gate.weight.zero_()
            layer.gate.weight[0] = 4.0  # positive inputs: expert 0 always wins, the second choice varies
            layer.gate.weight[1:] = torch.randn(3, 32) * 0.05
            out, _ = layer(x)
            idx, w, _ = M.route(torch.nn.functional.linear(x, layer.gate.weight), k, 1.0)
        assert int(torch.bincount(idx.reshape(-1).long(), minlength=E)[0]) == T
        cap = M.expert_capacity(T, E, k, 1.25, drop)
        assert cap == (384 if drop else 512)  # ceil(1.25 * 2 * 512 / 4) = 320 -> whole 128-row tiles; dropless: every token
        assert torch.allclose(out, M.moe_ffn_reference(x, idx, w, layer.experts_w1, layer.experts_w2, cap), atol=1e-5)
        outs[drop] = out
        stats = layer.get_routing_stats()
        assert (stats["dropped_fraction"] > 0.1) == drop
    loop = torch.zeros_like(x)
    for e in range(E):  # the reference layer's per-expert loop: gather, FFN, index_add; nothing is dropped
        tok, kk = (idx.long() == e).nonzero(as_tuple=True)
        g, u = (x[tok] @ layer.experts_w1[e].t()).chunk(2, dim=-1)
        loop.index_add_(0, tok, ((torch.nn.functional.silu(g) * u) @ layer.experts_w2[e].t()) * w[tok, kk][:, None])
    assert torch.allclose(outs[False], loop, atol=1e-5)
    assert torch.allclose(outs[True][:384], loop[:384], atol=1e-5) and not torch.allclose(outs[True][384:], loop[384:], atol=1e-4)


def test_mod_processes_only_the_selected_fraction_per_sequence():
    cfg = ModelConfig(**BASE, use_mod=True, mod_capacity_factor=0.25)
    f = MoDFFN(cfg)
    for p in f.parameters():
        torch.nn.init.normal_(p, std=0.05)
    h = torch.randn(3, 16, 128)
    res = torch.zeros_like(h)
    out, aux = f(h, res)
    touched = (out.abs().sum(-1) > 0).sum(1)
    assert touched.tolist() == [4, 4, 4] and aux.item() > 0
    assert f.router.get_stats()["selected_ratio"] == pytest.approx(0.25)


def test_kv_cache_matches_full_forward():
    torch.manual_seed(0)
    m = DeepSeekTransformer(ModelConfig(**BASE, use_moe=True, num_experts=4, capacity_factor=8.0, drop_tokens=False)).eval()
    ids = torch.randint(0, 1000, (2, 12))
    with torch.no_grad():
        full = m(ids, return_aux_loss=False)
        cache = m.make_cache(2, 16)
        a = m(ids[:, :8], cache=cache, return_aux_loss=False)
        outs = [a]
        for t in range(8, 12):
            outs.append(m(ids[:, t:t + 1], cache=cache, return_aux_loss=False))
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-4)


def test_tiny_config_trains_twenty_steps():
    """Benchmark shape [0]: hidden 256, 4 layers, 8q/2kv heads, I 688, layers 1 and 3 MoE (4 experts, top-2), AdamW 3e-4."""
    from adaptivetrainingsystem_b200.parallel.zero import ShardedEngine
    cfg = ConfigPresets.get("tiny_cpu")
    torch.manual_seed(cfg.seed)
    m = DeepSeekTransformer(cfg.to_model_config())
    assert [b.ffn_kind for b in m.layers] == ["dense", "moe", "dense", "moe"]
    eng = ShardedEngine(m, lr=3e-4, zero_stage=0)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 8192, (4, 257), generator=g)
    losses = []
    for _ in range(20):
        out = m.forward_loss(ids[:, :-1], ids[:, 1:])
        out["loss"].backward()
        eng.step()
        losses.append(out["lm_loss"].item())
    assert losses[-1] < losses[0] - 0.5 and all(math.isfinite(l) for l in losses)


def test_decode_with_device_side_cache_counters_matches_python_counters():
    """The graph-replayable decode path (fill level and RoPE positions in device tensors) gives the same logits as the
    ordinary cached decode."""
    import torch
    from adaptivetrainingsystem_b200.config import ConfigPresets
    from adaptivetrainingsystem_b200.models.transformer import DeepSeekTransformer
    torch.manual_seed(3)
    cfg = ConfigPresets.tiny_cpu()
    model = DeepSeekTransformer(cfg.to_model_config()).eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 9))
    with torch.no_grad():
        c1, c2 = model.make_cache(2, 16), model.make_cache(2, 16)
        model(ids[:, :6], cache=c1, return_aux_loss=False)
        model(ids[:, :6], cache=c2, return_aux_loss=False)
        c2.enable_device_lengths()
        for t in range(6, 9):
            a = model(ids[:, t:t + 1], cache=c1, last_token_only=True, return_aux_loss=False)
            b = model(ids[:, t:t + 1], cache=c2, last_token_only=True, return_aux_loss=False)
            c2.device_advance()
            c2.length += 1
            assert torch.allclose(a, b, atol=1e-5), t
        assert c2.device_lengths.tolist() == [9, 9] and c1.length == 9


def test_router_z_loss_adds_to_the_auxiliary_loss_and_trains_the_gate():
    torch.manual_seed(0)
    base = dict(vocab_size=128, hidden_size=32, num_layers=1, num_heads=4, num_kv_heads=2, intermediate_size=64, seq_length=16,
                use_moe=True, num_experts=4, moe_top_k=2, routing_noise_std=0.0, load_balancing_weight=0.0)
    ids = torch.randint(0, 128, (2, 16))
    m0 = DeepSeekTransformer(ModelConfig(**base))
    m1 = DeepSeekTransformer(ModelConfig(**base, router_z_loss_weight=0.1))
    m1.load_state_dict(m0.state_dict())
    a0 = m0.forward_loss(ids, ids)["aux_loss"]
    out = m1.forward_loss(ids, ids)
    layer = m1.get_moe_layers()[0]
    with torch.no_grad():
        h = m1.layers[0].post_attn_norm(m1.layers[0].self_attn(m1.layers[0].input_norm(m1.embed_tokens(ids) * (32 ** 0.5 if m1.config.use_stable_embedding else 1.0)),
                                                               m1.embed_tokens(ids) * (32 ** 0.5 if m1.config.use_stable_embedding else 1.0), m1.rope))
        want = 0.1 * torch.logsumexp(torch.nn.functional.linear(h.reshape(-1, 32), layer.gate.weight).float(), -1).pow(2).mean()
    assert float(a0) == 0.0 and abs(float(out["aux_loss"]) - float(want)) < 1e-4 * max(1.0, float(want))
    out["loss"].backward()
    assert layer.gate.weight.grad is not None and float(layer.gate.weight.grad.abs().sum()) > 0


def test_generation_without_kv_cache_matches_cached_generation():
    """``use_kv_cache=False`` (the reference's loop: the whole sequence again for every token) gives the tokens of the cached
    engine; a cache dtype the engine does not hold is refused."""
    import pytest
    from adaptivetrainingsystem_b200.inference import GenerationEngine, SamplingParams
    torch.manual_seed(0)
    cfg = ModelConfig(vocab_size=128, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128, seq_length=64)
    model = DeepSeekTransformer(cfg).eval()
    ids = torch.randint(0, 128, (2, 9))
    params = SamplingParams.from_mode("greedy", max_new_tokens=7)
    cached = GenerationEngine(model).generate(ids, params)
    plain = GenerationEngine(model, use_kv_cache=False).generate(ids, params)
    assert torch.equal(cached["tokens"], plain["tokens"]) and plain["kv_cache"] is False and plain["steps"] == 7
    with pytest.raises(ValueError):
        GenerationEngine(model, kv_cache_dtype="fp8")
    GenerationEngine(model, kv_cache_dtype="fp32")
