"""An unmodified Hugging Face Llama with every nn.Linear swapped for BlockInt8Linear: the way the reference is used.

    python examples/hf_llama_infer.py                      # Llama-2-7B shapes, random weights, batch 8, 512 + 32 tokens
    python examples/hf_llama_infer.py --layers 2 --hidden 256 --heads 4 --ffn 704 --vocab 512 --prompt 24 --decode 6

The reference's notebook (``examples/quantised_infer_llama.py/infer_llama.ipynb``) loads CodeLlama-7b-Python with
``AutoModelForCausalLM`` and applies the layer to it; there is no checkpoint here, so the model is built from a
``LlamaConfig`` of the same shapes with random weights.  Nothing of the model's code is touched:
``model.apply(replace_linear_with_blockwise_int8)`` swaps the 32 x 7 + 1 linear layers (``block_linear.py:16-32``),
``prepare_for_eval`` quantizes their weights once (``block_linear.py:125-128``) and drops the floating-point copies, and the
model's own ``generate`` runs the prompt and the greedy decode.  Prints one JSON line with the tokens per second of both
phases and of the same model before the swap (bf16 ``nn.Linear``).  This is the drop-in path: the time of a decode step is
mostly the Python of ``generate`` and the model's small torch kernels; ``examples/llama_infer.py`` is the driver built for
speed (static shapes, CUDA graphs, fused producer steps, tensor parallelism).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import block_linear_config as cfg  # noqa: E402
from block_linear import BlockInt8Linear, replace_linear_with_blockwise_int8  # noqa: E402


def build(a, dev):
    from transformers import LlamaConfig, LlamaForCausalLM
    config = LlamaConfig(hidden_size=a.hidden, intermediate_size=a.ffn, num_hidden_layers=a.layers, num_attention_heads=a.heads,
                         num_key_value_heads=a.heads, vocab_size=a.vocab, max_position_embeddings=a.prompt + a.decode + 8)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaForCausalLM(config).to(torch.bfloat16)
    return model.eval()


def timed_generate(model, ids, decode):
    """(prefill seconds, decode seconds, tokens): the prompt alone, then prompt + `decode` greedy tokens."""
    kw = dict(do_sample=False, pad_token_id=0)
    with torch.no_grad():
        model.generate(ids, max_new_tokens=3, min_new_tokens=3, **kw)     # lazy initialisation of both phases' kernels
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        model.generate(ids, max_new_tokens=1, **kw)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        t0 = time.perf_counter()
        out = model.generate(ids, max_new_tokens=decode, min_new_tokens=decode, **kw)
        torch.cuda.synchronize()
        t_all = time.perf_counter() - t0
    return t_prefill, max(t_all - t_prefill, 1e-9), out[:, ids.shape[1]:]


def run(a, dev):
    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = a.block, torch.bfloat16
    model = build(a, dev)
    ids = torch.randint(0, a.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(4000)).to(dev)
    res = {"model": f"transformers LlamaForCausalLM {a.layers}x{a.hidden} ffn {a.ffn} vocab {a.vocab}, random init",
           "batch": a.batch, "prompt": a.prompt, "decode": a.decode}
    if not a.skip_dense:
        tp, td, toks = timed_generate(model, ids, a.decode)
        res["bf16_dense"] = {"prefill_tokens_per_s": a.batch * a.prompt / tp, "decode_tokens_per_s": a.batch * (a.decode - 1) / td,
                             "first_tokens": toks[0, :8].tolist()}
    model.apply(replace_linear_with_blockwise_int8)                        # the reference's patcher, module by module
    layers = [m for m in model.modules() if isinstance(m, BlockInt8Linear)]
    for m in layers:
        m.prepare_for_eval(drop_weight=True)                               # int8 weights only: 7 GB instead of 13.5 GB at 7B
    torch.cuda.empty_cache()
    tp, td, toks = timed_generate(model, ids, a.decode)
    res["int8"] = {"linear_layers_replaced": len(layers), "prefill_tokens_per_s": a.batch * a.prompt / tp,
                   "decode_tokens_per_s": a.batch * (a.decode - 1) / td, "first_tokens": toks[0, :8].tolist(),
                   "weights_gb": sum(m.W_int8.numel() + 4 * m.state_W.numel() for m in layers) / 1e9}
    from blockwise_int8_linear_b200 import _lib
    _lib.device_status()
    return res, model


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--decode", type=int, default=32)
    ap.add_argument("--block", type=int, default=64)
    ap.add_argument("--skip-dense", dest="skip_dense", action="store_true", help="do not time the bf16 model before the swap")
    a = ap.parse_args()
    res, _ = run(a, torch.device("cuda"))
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
