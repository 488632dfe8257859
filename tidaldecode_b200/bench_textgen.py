"""End-to-end decode latency of a random-init Llama on one GPU — the protocol of the reference's
scripts/bench_textgen.py:40-101 (prefill a context, then decode_len greedy steps, report the mean
per-token latency), with the step replayed as a CUDA graph.

    python -m tidaldecode_b200.bench_textgen --model llama2-7b --context_len 32768 --decode_len 256 --token_budget 256

Prints one JSON line per run.  Weights are random (std 0.02), inputs random token ids: the reference
feeds random embeddings to a random-init model as well (bench_textgen.py:60-89).
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from .llama import LlamaConfig, LlamaForCausalLM
from .runtime import GraphDecoder

MODELS = {
    # name: (hidden, ffn, layers, heads, kv_heads, vocab, theta, dtype)
    "llama2-7b": (4096, 11008, 32, 32, 32, 32000, 1e4, torch.float16),
    "llama3-8b": (4096, 14336, 32, 32, 8, 128256, 5e5, torch.bfloat16),
    "llama-1b": (2048, 5632, 22, 32, 4, 32000, 1e4, torch.float16),       # small enough to profile (2.2 GB of weights)
    "tiny": (256, 688, 4, 4, 4, 1024, 1e4, torch.float32),
}


def build(name, selection_layers, head_reduce, force_last):
    h, f, L, H, Hkv, V, theta, dtype = MODELS[name]
    cfg = LlamaConfig(vocab_size=V, hidden_size=h, intermediate_size=f, num_hidden_layers=L, num_attention_heads=H,
                      num_key_value_heads=Hkv, rope_theta=theta, selection_layers=tuple(selection_layers),
                      head_reduce=head_reduce, force_last_token=force_last)
    torch.manual_seed(0)
    with torch.device("cuda"):
        m = LlamaForCausalLM(cfg).to(dtype)
    for p in m.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.02)
    return m.eval(), dtype


@torch.inference_mode()
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=sorted(MODELS), default="llama2-7b")
    ap.add_argument("--context_len", type=int, default=32768)
    ap.add_argument("--decode_len", type=int, default=256)
    ap.add_argument("--token_budget", type=int, default=256)
    ap.add_argument("--selection_layers", type=int, nargs="*", default=[2, 13])
    ap.add_argument("--head_reduce", choices=["none", "sum"], default="none")
    ap.add_argument("--full", action="store_true", help="full attention in every layer (budget = context)")
    ap.add_argument("--iteration", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded in lockstep; more than one implies --random_cache")
    ap.add_argument("--random_cache", action="store_true",
                    help="skip prefill: decode from KV caches filled with random values (prefill takes one sequence at a time)")
    ap.add_argument("--torch_linear", action="store_true", help="projections, norms and activations as separate torch/cuBLAS ops")
    a = ap.parse_args()
    sel = [] if a.full else a.selection_layers
    m, dtype = build(a.model, sel, a.head_reduce, True)
    max_len = a.context_len + a.decode_len + 8
    rt = GraphDecoder(m, max_seq_len=max_len, token_budget=a.token_budget, dtype=dtype, fused_linear=not a.torch_linear,
                      batch_size=a.batch)
    g = torch.Generator().manual_seed(0)
    for it in range(a.iteration):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if a.batch > 1 or a.random_cache:
            rt.start_from_cache(a.context_len, torch.randint(0, m.vocab_size, (a.batch,), generator=g))
            kv = rt.c.kv_cache
            for layer in range(kv.pool.num_layers):              # N(0,1) keys and values, a layer at a time
                kv.pool.buf[layer].normal_()
        else:
            prompt = torch.randint(0, m.vocab_size, (1, a.context_len), generator=g)
            rt.prefill(prompt)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        rt.decode(2)                                            # eager step + capture + one replay
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        toks = rt.decode(a.decode_len - 2)
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        n = a.decode_len - 2
        print(json.dumps({
            "model": a.model, "batch": a.batch, "context_len": a.context_len, "decode_len": a.decode_len,
            "token_budget": None if a.full else a.token_budget, "selection_layers": sel, "head_reduce": a.head_reduce, "fused_linear": rt.fused_linear,
            "prefill_s": round(t_prefill, 3), "decode_ms_per_token_device": round(e0.elapsed_time(e1) / n, 4),
            "decode_ms_per_token_wall": round(wall * 1e3 / n, 4), "tokens_per_s": round(a.batch * n / wall, 1),
            "status": rt.c.workspace.status() | int(rt.lin_status.item()), "last_tokens": toks[0, -4:].tolist()}))


if __name__ == "__main__":
    main()
