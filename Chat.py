#!/usr/bin/env python
"""Interactive chat / batch generation from a checkpoint.

    python Chat.py --checkpoint experiments/run/checkpoints/checkpoint_final.pt [--mode standard] [--prompt "..."]

Loads single-file checkpoints under any of the keys ``model_state_dict | module | state_dict | model`` and infers the
architecture from the tensor names when no config is stored (reference ``Chat.py:132-298``); generation uses the KV-cache
engine.  Slash commands: /mode <name>, /temp <x>, /tokens <n>, /reset, /stats, /quit (reference ``Chat.py:671-707``)."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

from adaptivetrainingsystem_b200.config import ModelConfig  # noqa: E402
from adaptivetrainingsystem_b200.data.tokenizer import ConversationTokenizer  # noqa: E402
from adaptivetrainingsystem_b200.inference import GENERATION_MODES, GenerationEngine, SamplingParams  # noqa: E402
from adaptivetrainingsystem_b200.models import DeepSeekTransformer  # noqa: E402
from adaptivetrainingsystem_b200.training.checkpoint import MODEL_KEYS  # noqa: E402


def infer_config_from_state_dict(sd) -> ModelConfig:
    """Architecture from parameter names and shapes."""
    vocab, hidden = sd["embed_tokens.weight"].shape
    layers = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
    q = sd["layers.0.self_attn.q_proj.weight"].shape[0]
    kv = sd["layers.0.self_attn.k_proj.weight"].shape[0]
    moe_layers = sorted({int(k.split(".")[1]) for k in sd if ".ffn.gate.weight" in k})
    mod_layers = sorted({int(k.split(".")[1]) for k in sd if ".ffn.router.router.weight" in k})
    head_dim = 128 if q % 128 == 0 and hidden >= 2048 else 64 if q % 64 == 0 else 32
    n_exp = sd[f"layers.{moe_layers[0]}.ffn.gate.weight"].shape[0] if moe_layers else 8
    if moe_layers:
        inter = sd[f"layers.{moe_layers[0]}.ffn.experts.0.gate_up_proj.weight"].shape[0] // 2
    else:
        inter = sd["layers.0.ffn.gate_up_proj.weight"].shape[0] // 2
    tied = "lm_head.weight" not in sd or sd["lm_head.weight"].data_ptr() == sd["embed_tokens.weight"].data_ptr() or \
        torch.equal(sd["lm_head.weight"], sd["embed_tokens.weight"])
    return ModelConfig(vocab_size=vocab, hidden_size=hidden, num_layers=layers, num_heads=q // head_dim, num_kv_heads=kv // head_dim,
                       intermediate_size=inter, use_moe=bool(moe_layers), num_experts=n_exp, moe_layers=moe_layers or None,
                       use_mod=bool(mod_layers), mod_layers=mod_layers or None, tie_word_embeddings=tied)


def load_checkpoint_smart(path: str):
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    sd = next((ckpt[k] for k in MODEL_KEYS if isinstance(ckpt, dict) and k in ckpt), ckpt)
    mc = ckpt.get("model_config") if isinstance(ckpt, dict) else None
    cfg = ModelConfig.from_dict(mc) if mc else infer_config_from_state_dict(sd)
    return sd, cfg


class ChatInterface:
    def __init__(self, checkpoint: str, device: str = "auto", mode: str = "standard", quantize: str = None, quantized_file: str = None):
        self.device = torch.device("cuda" if (device == "auto" and torch.cuda.is_available()) else ("cpu" if device == "auto" else device))
        sd, cfg = load_checkpoint_smart(checkpoint)
        cfg.gradient_checkpointing = False
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.model = DeepSeekTransformer(cfg)
        self.model.load_state_dict({k: v for k, v in sd.items()}, strict=False)
        self.model = self.model.to(self.device, dtype).eval()
        if quantize:
            if self.device.type != "cuda" and quantize != "int4":
                raise SystemExit("--quantize fp8 / int8 needs a GPU: those paths run on the tensor-core GEMM")
            from types import SimpleNamespace
            from adaptivetrainingsystem_b200.training import QuantizationManager
            qm = QuantizationManager(SimpleNamespace(quantization_method=quantize, quantization_bits=4 if quantize == "int4" else 8))
            if quantize == "int4" and quantized_file and os.path.exists(quantized_file):
                # 4-bit copies written earlier (possibly GPTQ-calibrated): attach them and drop the bf16 projections
                qm.load_quantized(self.model, quantized_file, release_originals=True)
            else:
                qm.quantize_model(self.model)
                if quantize == "int4" and quantized_file:
                    qm.save_quantized(self.model, quantized_file)
        self.tokenizer = ConversationTokenizer()
        self.engine = GenerationEngine(self.model, self.tokenizer, use_kv_cache=bool(getattr(cfg, "use_kv_cache", True)))
        self.params = SamplingParams.from_mode(mode, max_new_tokens=min(256, max(cfg.seq_length // 2, 1)),
                                               stop_token_ids=(self.tokenizer.special_tokens["<|im_end|>"], self.tokenizer.eos_token_id))
        self.history = []

    def _format_prompt(self, user_text: str):
        msgs = self.history + [{"role": "user", "content": user_text}]
        enc = self.tokenizer.encode_conversation(msgs, max_length=max(self.model.config.seq_length - self.params.max_new_tokens, 8),
                                                 truncation="keep_system", add_generation_prompt=True)
        return torch.tensor([enc["input_ids"]], dtype=torch.long, device=self.device).clamp(max=self.model.config.vocab_size - 1)

    def respond(self, user_text: str) -> str:
        ids = self._format_prompt(user_text)
        res = self.engine.generate(ids, self.params)
        text = self.tokenizer.decode(res["tokens"][0].tolist())
        self.history += [{"role": "user", "content": user_text}, {"role": "assistant", "content": text}]
        return text

    def respond_many(self, user_texts, max_batch: int = 16):
        """Independent single-turn prompts served together: continuous batching over ``max_batch`` cache rows (GPU only)."""
        from adaptivetrainingsystem_b200.inference import ContinuousBatcher
        saved, self.history = self.history, []
        try:
            prompts = [self._format_prompt(t)[0].tolist() for t in user_texts]
        finally:
            self.history = saved
        rows = max(len(p) for p in prompts) + self.params.max_new_tokens
        batcher = ContinuousBatcher(self.engine, max_batch=min(max_batch, len(prompts)), max_len=rows, params=self.params)
        return [self.tokenizer.decode(t) for t in batcher.run(prompts)]

    def command(self, line: str) -> bool:
        cmd, *rest = line[1:].split()
        if cmd in ("quit", "exit"):
            return False
        if cmd == "mode" and rest and rest[0] in GENERATION_MODES:
            for k, v in GENERATION_MODES[rest[0]].items():
                setattr(self.params, k, v)
        elif cmd == "temp" and rest:
            self.params.temperature = float(rest[0])
        elif cmd == "tokens" and rest:
            self.params.max_new_tokens = int(rest[0])
        elif cmd == "reset":
            self.history = []
        elif cmd == "stats":
            print(self.engine.stats)
        else:
            print("commands: /mode <%s> /temp x /tokens n /reset /stats /quit" % "|".join(GENERATION_MODES))
        return True

    def run(self) -> None:
        print("chat ready; /quit to leave")
        while True:
            try:
                line = input("> ").strip()
            except (EOFError, KeyboardInterrupt):
                break
            if not line:
                continue
            if line.startswith("/"):
                if not self.command(line):
                    break
                continue
            print(self.respond(line))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--mode", default="standard", choices=list(GENERATION_MODES))
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--quantize", default=None, choices=["fp8", "int8", "int4"], help="post-training quantisation of the projection weights")
    ap.add_argument("--quantized-file", default=None,
                    help="with --quantize int4: load the packed 4-bit copies from this file if it exists (the bf16 projections are freed), else write them there")
    ap.add_argument("--prompts-file", default=None, help="one prompt per line, answered together by continuous batching")
    ap.add_argument("--max-batch", type=int, default=16)
    a = ap.parse_args()
    chat = ChatInterface(a.checkpoint, a.device, a.mode, a.quantize, a.quantized_file)
    if a.prompts_file:
        with open(a.prompts_file) as f:
            lines = [l.strip() for l in f if l.strip()]
        for q, ans in zip(lines, chat.respond_many(lines, a.max_batch)):
            print(f"> {q}\n{ans}\n")
    elif a.prompt:
        print(chat.respond(a.prompt))
    else:
        chat.run()
