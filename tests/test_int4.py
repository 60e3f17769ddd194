"""Weight-only 4-bit layers: packed format, GPTQ against round-to-nearest, the manager on CPU, and the kernels against the
fp32 product of the dequantised weight on the GPU."""
from types import SimpleNamespace

import pytest
import torch

from adaptivetrainingsystem_b200.config import ModelConfig
from adaptivetrainingsystem_b200.models import DeepSeekTransformer
from adaptivetrainingsystem_b200.ops import int4


def test_packed_format_round_trip_and_nibble_positions():
    torch.manual_seed(0)
    N, K = 48, 192
    q = torch.randint(0, 16, (N, K), dtype=torch.uint8)
    packed = int4.pack(q)
    assert packed.shape == (K // 64, N // 16, 32, 4) and packed.dtype == torch.int32
    assert torch.equal(int4.unpack(packed), q)
    # the documented position of a code: tile T, super-step S, lane 4 g + t, word j, nibble i
    for T, S, g, t, j, i in [(0, 0, 0, 0, 0, 0), (2, 1, 5, 3, 2, 7), (1, 2, 7, 1, 3, 4), (0, 1, 3, 2, 1, 3)]:
        word = int(packed[S, T, 4 * g + t, j]) & 0xFFFFFFFF
        row = 16 * T + g + 8 * (i & 1)
        col = 64 * S + 16 * t + 4 * j + 2 * ((i >> 1) & 1) + (i >> 2)
        assert (word >> (4 * i)) & 15 == int(q[row, col])
    scale = torch.rand(N, 3).to(torch.bfloat16).float() + 0.01
    zero = torch.randint(0, 16, (N, 3)).float()
    meta = int4.pack_meta(scale.to(torch.bfloat16).float(), zero)
    s2, z2 = int4.unpack_meta(meta)
    assert meta.shape == (3, N) and torch.equal(s2, scale.to(torch.bfloat16).float()) and torch.equal(z2, zero)


def test_round_to_nearest_error_is_within_half_a_step():
    torch.manual_seed(1)
    w = torch.randn(32, 256) * 0.1
    q, scale, zero = int4.quantize_rtn(w, 128)
    wd = int4.dequantize_reference(int4.pack(q), int4.pack_meta(scale, zero), 128).float()
    step = scale.repeat_interleave(128, dim=1)
    assert ((w - wd).abs() <= 0.5 * step + 2.0 ** -8 * w.abs() + 1e-6).all()   # half a step plus the bf16 rounding of the value


def test_gptq_beats_round_to_nearest_on_correlated_inputs():
    torch.manual_seed(2)
    N, K = 64, 256
    w = torch.randn(N, K) * 0.05
    x = torch.randn(512, 16) @ torch.randn(16, K) + 0.3 * torch.randn(512, K)
    H = x.t() @ x

    def err(q, s, z):
        wd = int4.dequantize_reference(int4.pack(q), int4.pack_meta(s, z), 128).float()
        return ((x @ (w - wd).t()) ** 2).sum().item()

    e_rtn = err(*int4.quantize_rtn(w, 128))
    e_gptq = err(*int4.gptq_quantize(w, H, 128))
    assert e_gptq < 0.5 * e_rtn, (e_gptq, e_rtn)


def test_gptq_act_order_helps_when_input_channels_differ_in_scale():
    """Channels of very different magnitude: fixing the heavy ones first (static groups, stored layout unchanged) lowers the
    output error again; the codes still unpack to [N, K] with groups of consecutive channels."""
    torch.manual_seed(2)
    N, K = 64, 512
    w = torch.randn(N, K) * 0.05
    x = (torch.randn(1024, 16) @ torch.randn(16, K) + 0.3 * torch.randn(1024, K)) * torch.exp(torch.randn(K) * 1.5)
    H = x.t() @ x

    def err(q, s, z):
        assert q.shape == (N, K) and s.shape == (N, K // 128) and int(q.max()) <= 15
        wd = int4.dequantize_reference(int4.pack(q), int4.pack_meta(s, z), 128).float()
        return ((x @ (w - wd).t()) ** 2).sum().item()

    e_plain = err(*int4.gptq_quantize(w, H, 128))
    e_act = err(*int4.gptq_quantize(w, H, 128, act_order=True))
    assert e_act < 0.6 * e_plain, (e_act, e_plain)


def test_manager_quantises_projections_to_4_bits_cpu():
    """Through the manager on CPU (PyTorch definitions): GPTQ refuses to run uncalibrated; after calibration every projection
    gets a Hessian (the down projection's through the two-step MLP), the head stays in bf16, and the logits stay close."""
    from adaptivetrainingsystem_b200.training.precision import QuantizationManager
    torch.manual_seed(0)
    cfg = ModelConfig(vocab_size=256, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=256, seq_length=32,
                      tie_word_embeddings=False)
    ids = torch.randint(0, 256, (4, 32))
    try:
        model = DeepSeekTransformer(cfg)
        with torch.no_grad():
            ref = model(ids, return_aux_loss=False)
        with pytest.raises(RuntimeError):
            QuantizationManager(SimpleNamespace(quantization_method="gptq", quantization_bits=4)).quantize_model(model)
        qm = QuantizationManager(SimpleNamespace(quantization_method=None, quantization_bits=4))
        assert qm.method == "int4"
        n_h = qm.calibrate(model, [ids, torch.randint(0, 256, (4, 32))])
        assert n_h == 8                                     # qkv, o, gate_up, down of both layers (the head stays in bf16: not observed)
        qm.quantize_model(model)
        st = qm.status()
        assert st["applied"] and st["tensors"] == 8 and st["gptq_weights"] == 8
        assert int4.lookup(model.lm_head_weight) is None and int4.lookup(model.layers[0].ffn.down_proj) is not None
        with torch.no_grad():
            out = model(ids, return_aux_loss=False)
        rel = ((out - ref).norm() / ref.norm()).item()
        assert 0.0 < rel < 0.2, rel
        # a changed weight no longer matches its registered copy: back to the unquantised product
        model.layers[0].self_attn.o_proj.data.mul_(1.0)
        model.layers[0].self_attn.o_proj.add_(0.0)
        assert int4.lookup(model.layers[0].self_attn.o_proj) is None
    finally:
        int4.set_enabled(False)
        int4.clear()


def test_symmetric_codes_and_block_by_block_gptq_cpu():
    """``sym``: zero point 8 everywhere and a range that covers -max |w| .. max |w|.  Block-by-block GPTQ: every projection gets
    GPTQ codes, only one block's Hessians exist at a time, and the logits stay as close as with one-shot calibration."""
    from adaptivetrainingsystem_b200.training.precision import QuantizationManager
    torch.manual_seed(3)
    w = torch.randn(32, 256) * 0.1
    q, scale, zero = int4.quantize_rtn(w, 128, sym=True)
    assert (zero == 8).all()
    wd = int4.dequantize_reference(int4.pack(q), int4.pack_meta(scale, zero), 128).float()
    assert ((w - wd).abs() <= 0.5 * scale.repeat_interleave(128, dim=1) * 1.05 + 2.0 ** -8 * w.abs() + 1e-6).all()   # the bf16 scale may fall 0.2 % short of max / 7.5
    cfg = ModelConfig(vocab_size=256, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=256, seq_length=32,
                      tie_word_embeddings=False)
    ids = [torch.randint(0, 256, (4, 32)) for _ in range(2)]
    errs = {}
    for mode in ("one_shot", "sequential"):
        torch.manual_seed(0)
        model = DeepSeekTransformer(cfg)
        with torch.no_grad():
            ref = model(ids[0], return_aux_loss=False)
        try:
            qm = QuantizationManager(SimpleNamespace(quantization_method="gptq", quantization_bits=4, quantization_symmetric=True))
            assert qm.symmetric
            if mode == "one_shot":
                qm.calibrate(model, ids)
                qm.quantize_model(model)
            else:
                qm.quantize_sequential(model, ids)
                assert int4.hessian_count() == 0 and int4.enabled()
            assert qm.status()["tensors"] == 8 and qm.status()["gptq_weights"] == 8
            _, zero_l = int4.unpack_meta(int4.lookup(model.layers[1].ffn.down_proj)[1])
            assert (zero_l == 8).all()
            with torch.no_grad():
                out = model(ids[0], return_aux_loss=False)
            errs[mode] = ((out - ref).norm() / ref.norm()).item()
        finally:
            int4.set_enabled(False)
            int4.clear()
    assert 0.0 < errs["sequential"] < 0.25 and errs["sequential"] < 1.5 * errs["one_shot"], errs


def test_saved_4bit_copies_serve_a_fresh_model_without_its_bf16_projections(tmp_path):
    """save_quantized -> a fresh model of the same architecture (other projection values) -> load_quantized with the bf16
    storage released: the same logits as the model that was quantised, and the projections hold no storage of their own."""
    from adaptivetrainingsystem_b200.training.precision import QuantizationManager
    cfg = ModelConfig(vocab_size=256, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=256, seq_length=32,
                      tie_word_embeddings=False)
    ids = torch.randint(0, 256, (2, 32))
    path = str(tmp_path / "q4.pt")
    try:
        torch.manual_seed(0)
        model = DeepSeekTransformer(cfg)
        qm = QuantizationManager(SimpleNamespace(quantization_method="int4", quantization_bits=4))
        with pytest.raises(RuntimeError):
            qm.save_quantized(model, path)                       # nothing quantised yet
        qm.quantize_model(model)
        assert qm.save_quantized(model, path) == 8
        with torch.no_grad():
            ref = model(ids, return_aux_loss=False)
        kept = {n: p.detach().clone() for n, p in model.named_parameters() if p.dim() != 2 or "lm_head" in n or "embed" in n}
        int4.set_enabled(False)
        int4.clear()
        torch.manual_seed(1)
        fresh = DeepSeekTransformer(cfg)                          # other projections; head, embeddings and norms copied over
        with torch.no_grad():
            for n, p in fresh.named_parameters():
                if n in kept:
                    p.copy_(kept[n])
        qm2 = QuantizationManager(SimpleNamespace(quantization_method=None, quantization_bits=None))
        assert qm2.load_quantized(fresh, path, release_originals=True) == 8
        assert qm2.status()["method"] == "int4" and qm2.released_bytes == sum(p.numel() * 4 for n, p in model.named_parameters()
                                                                              if p.dim() == 2 and "lm_head" not in n and "embed" not in n)
        proj = fresh.layers[0].ffn.down_proj
        assert proj.shape == (128, 256) and proj.stride() == (0, 0) and proj.untyped_storage().nbytes() <= 8
        with torch.no_grad():
            out = fresh(ids, return_aux_loss=False)
        assert torch.equal(out, ref)
        assert qm2.release_originals(fresh) == 0                 # nothing left to free
        with pytest.raises(RuntimeError):
            torch.save({"format": "other"}, path)
            qm2.load_quantized(fresh, path)
    finally:
        int4.set_enabled(False)
        int4.clear()


def test_export_for_inference_writes_a_checkpoint_the_chat_loader_reads(tmp_path):
    """The exported file goes through the chat entry point's loader into an identical model; the int4 export adds the packed
    copies (GPTQ block by block with calibration batches) and leaves the exporting model unquantised and trainable."""
    import importlib.util
    import os
    from adaptivetrainingsystem_b200.training.precision import QuantizationManager
    from adaptivetrainingsystem_b200.utils import export_for_inference
    spec = importlib.util.spec_from_file_location("chat_entry", os.path.join(os.path.dirname(os.path.dirname(__file__)), "Chat.py"))
    chat = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(chat)
    torch.manual_seed(0)
    cfg = ModelConfig(vocab_size=256, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=256, seq_length=32,
                      tie_word_embeddings=False)
    model = DeepSeekTransformer(cfg)
    ids = torch.randint(0, 256, (2, 32))
    path = str(tmp_path / "serve.pt")
    try:
        info = export_for_inference(model, path, dtype=torch.float32, quantize="int4", calibration_batches=[ids])
        assert info["quantized_tensors"] == 8 and info["gptq_tensors"] == 8 and info["quantized_bytes"] < info["checkpoint_bytes"] / 4
        assert not int4.enabled() and all(p.requires_grad for p in model.parameters())
        with torch.no_grad():
            ref = model(ids, return_aux_loss=False)
        sd, cfg2 = chat.load_checkpoint_smart(path)
        served = DeepSeekTransformer(cfg2)
        served.load_state_dict(sd, strict=False)
        served.eval()
        with torch.no_grad():
            assert torch.equal(served(ids, return_aux_loss=False), ref)
        qm = QuantizationManager(SimpleNamespace(quantization_method=None, quantization_bits=None))
        assert qm.load_quantized(served, info["quantized"], release_originals=True) == 8
        with torch.no_grad():
            out = served(ids, return_aux_loss=False)
        assert 0.0 < ((out - ref).norm() / ref.norm()).item() < 0.1
        with pytest.raises(ValueError):
            export_for_inference(model, path, quantize="fp8")
    finally:
        int4.set_enabled(False)
        int4.clear()


def test_chat_serves_saved_4bit_copies_cpu(tmp_path):
    """The chat entry point with ``--quantize int4 --quantized-file``: the first start writes the packed copies, the second one
    attaches them, frees the projections and answers with the same tokens (greedy)."""
    import importlib.util
    import os
    from adaptivetrainingsystem_b200.utils import export_for_inference
    spec = importlib.util.spec_from_file_location("chat_entry2", os.path.join(os.path.dirname(os.path.dirname(__file__)), "Chat.py"))
    chat = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(chat)
    torch.manual_seed(0)
    cfg = ModelConfig(vocab_size=512, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=256, seq_length=128,
                      tie_word_embeddings=False)
    ckpt, qfile = str(tmp_path / "m.pt"), str(tmp_path / "m.int4")
    export_for_inference(DeepSeekTransformer(cfg), ckpt, dtype=torch.float32)
    answers = []
    try:
        for start in range(2):
            c = chat.ChatInterface(ckpt, device="cpu", mode="greedy", quantize="int4", quantized_file=qfile)
            c.params.max_new_tokens = 6
            answers.append(c.engine.generate(c._format_prompt("hello there"), c.params)["tokens"][0].tolist())
            assert os.path.exists(qfile)
            assert (c.model.layers[0].ffn.down_proj.stride() == (0, 0)) == (start == 1)
            int4.set_enabled(False)
            int4.clear()
        assert answers[0] == answers[1] and len(answers[0]) == 6
    finally:
        int4.set_enabled(False)
        int4.clear()


# ------------------------------------------------------------------------------------------------------------------------- GPU
def _packed(N, K, group, dev, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.05
    q, scale, zero = int4.quantize_rtn(w, group)
    return int4.pack(q).to(dev), int4.pack_meta(scale, zero).to(dev)


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,group", [(64, 256, 128), (2560, 2048, 128), (1024, 5632, 64)])
def test_dequant_kernel_matches_reference_bit_for_bit(N, K, group):
    dev = torch.device("cuda")
    packed, meta = _packed(N, K, group, dev, 3)
    ref = int4.dequantize_reference(packed.cpu(), meta.cpu(), group)
    out = int4.dequantize(packed, meta, group)
    assert out.shape == (N, K) and torch.equal(out.cpu(), ref)
    # into a wider matrix (row pitch != K)
    wide = torch.zeros(N, K + 64, dtype=torch.bfloat16, device=dev)
    int4.dequantize(packed, meta, group, out=wide[:, :K])
    assert torch.equal(wide[:, :K].cpu(), ref) and float(wide[:, K:].abs().sum()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,group", [(1, 64, 256, 128), (3, 2560, 2048, 128), (8, 2048, 5632, 128), (5, 32000, 2048, 128), (13, 512, 1024, 64),
                                           (16, 28672, 1024, 256), (9, 2560, 2048, 128)])
def test_gemv_kernel_matches_fp32_product(M, N, K, group):
    """One tile per CTA (small N), two tiles per CTA (N / 32 >= 592), one and two token tiles, with and without the residual."""
    dev = torch.device("cuda")
    torch.manual_seed(M)
    packed, meta = _packed(N, K, group, dev, 4)
    wd = int4.dequantize_reference(packed.cpu(), meta.cpu(), group).float().to(dev)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    add = torch.randn(M, N, device=dev).to(torch.bfloat16)
    ref = x.float() @ wd.t()
    tol = 2.0 ** -7 * ref.abs().max().item() + 1e-3
    out = int4.gemv(x, packed, meta, group)
    assert out.shape == (M, N) and (out.float() - ref).abs().max().item() < tol
    out = int4.gemv(x, packed, meta, group, add=add)
    assert (out.float() - (ref + add.float())).abs().max().item() < tol + 2.0 ** -7 * add.abs().max().item()
    # rows of a wider activation buffer (row pitch != K)
    xw = torch.randn(M, K + 64, device=dev).to(torch.bfloat16)
    out = int4.gemv(xw[:, :K], packed, meta, group)
    assert (out.float() - xw[:, :K].float() @ wd.t()).abs().max().item() < tol


@pytest.mark.gpu
@pytest.mark.parametrize("M,inter,K", [(1, 128, 256), (4, 5632, 2048), (8, 14336, 1024), (12, 5632, 2048)])
def test_gemv_kernel_swiglu_epilogue(M, inter, K):
    dev = torch.device("cuda")
    torch.manual_seed(7)
    packed, meta = _packed(2 * inter, K, 128, dev, 5)
    wd = int4.dequantize_reference(packed.cpu(), meta.cpu(), 128).float().to(dev)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    gu = (x.float() @ wd.t()).to(torch.bfloat16).float()
    ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    out = int4.gemv(x, packed, meta, 128, swiglu=True)
    assert out.shape == (M, inter)
    # a gate or up value that lands on the other side of a bf16 rounding boundary moves the product by one bf16 step of it
    assert (out.float() - ref).abs().max().item() < 2.0 ** -6 * ref.abs().max().item() + 1e-3


@pytest.mark.gpu
def test_int4_model_matches_its_dequantised_weights():
    """Weights replaced by their dequantised 4-bit values give the oracle.  The 4-bit kernels (a prompt through dequantise +
    tcgen05 GEMM, eight rows and graph-replayed decode steps through the streaming kernel) must reproduce its logits, and every
    token the quantised engine generates greedily must be the oracle's choice up to a near tie."""
    from adaptivetrainingsystem_b200.inference.engine import GenerationEngine, SamplingParams
    from adaptivetrainingsystem_b200.training.precision import QuantizationManager
    dev = torch.device("cuda")
    torch.manual_seed(0)
    cfg = ModelConfig(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2, intermediate_size=1024, seq_length=256,
                      tie_word_embeddings=False)
    model = DeepSeekTransformer(cfg).to(dev, torch.bfloat16).eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 48), device=dev)
    try:
        qm = QuantizationManager(SimpleNamespace(quantization_method="int4", quantization_bits=4))
        assert qm.calibrate(model, [torch.randint(0, cfg.vocab_size, (4, 128), device=dev)]) >= 8
        qm.quantize_model(model)
        assert qm.status()["tensors"] == 8 and qm.status()["gptq_weights"] >= 4
        with torch.no_grad():
            out_q = model(ids, return_aux_loss=False).float()                       # 96 rows: dequantise + tcgen05 GEMM
            out_q1 = model(ids[:1, :8], return_aux_loss=False).float()              # 8 rows: the streaming kernel
        gen_q = GenerationEngine(model, max_batch=2).generate(ids, SamplingParams.from_mode("greedy", max_new_tokens=16))["tokens"].to(dev)
        assert gen_q.shape == (2, 16)
        int4.set_enabled(False)
        with torch.no_grad():
            copies = {name: int4.lookup(p) for name, p in model.named_parameters()}
            for name, p in model.named_parameters():
                if copies[name] is not None:
                    p.copy_(int4.dequantize(*copies[name]))
            out_d = model(ids, return_aux_loss=False).float()
            out_d1 = model(ids[:1, :8], return_aux_loss=False).float()
            lg = model(torch.cat([ids, gen_q], 1), return_aux_loss=False).float()[:, 47:63]     # the oracle's logits for every generated token
        assert ((out_q - out_d).norm() / out_d.norm()).item() < 2e-2
        assert ((out_q1 - out_d1).norm() / out_d1.norm()).item() < 2e-2
        gap = lg.max(-1).values - lg.gather(-1, gen_q[..., None]).squeeze(-1)
        assert gap.max().item() < 0.15 * lg.std().item(), (gap.max().item(), lg.std().item())
    finally:
        int4.set_enabled(False)
        int4.clear()
