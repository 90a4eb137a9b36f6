"""Reference model families for the training entry points and benchmarks: a GPT-2-style decoder
(LayerNorm, learned positions, GELU MLP) and a Llama-style decoder (RMSNorm, RoPE, SwiGLU, grouped
KV heads).  They exist to exercise the optimizers on the shapes named by the benchmark configs; the
attention core is ``torch.nn.functional.scaled_dot_product_attention``."""

from .gpt import GPT, GPTConfig, gpt2_small, gpt_350m
from .graphs import graph_forward_backward
from .llama import Llama, LlamaConfig, llama_1p3b, llama3_8b


def split_param_groups(model):
    """``(matrices, rest)``: 2-D weights of the transformer blocks go to a matrix optimizer (Muon,
    SOAP, PSGD); embeddings, output head, norms and biases go to an element-wise one."""
    mats, rest = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        in_block = ".blocks." in f".{name}" or ".layers." in f".{name}"
        (mats if (p.ndim >= 2 and in_block) else rest).append(p)
    return mats, rest


__all__ = [
    "GPT", "GPTConfig", "gpt2_small", "gpt_350m", "Llama", "LlamaConfig", "llama_1p3b", "llama3_8b",
    "split_param_groups", "graph_forward_backward",
]  # fmt: skip
