"""Model families assembled from the library's modules.

Decoder-only (all share ``LlamaModel``'s block, tensor + sequence parallel layouts, fused cross entropy and decoding
on the key/value cache): ``llama``, ``mistral`` (sliding window), ``gemma`` (GeGLU, tied head), ``qwen`` (per-head
q/k norms), ``gpt`` (LayerNorm, learned positions), ``mixtral`` (routed experts, expert parallel).
Encoder: ``bert``.  Encoder-decoder: ``t5``.  ``hf`` converts Hugging Face checkpoints; ``generation`` is the
decoding loop.  Submodules are imported on first use so that ``import transformerengine_b200`` stays light.
"""
import importlib

_LAZY = {
    "LlamaConfig": "llama", "LlamaModel": "llama",
    "MistralConfig": "mistral", "MistralModel": "mistral",
    "GemmaConfig": "gemma", "GemmaModel": "gemma",
    "Qwen3Config": "qwen", "Qwen3Model": "qwen",
    "GPTConfig": "gpt", "GPTModel": "gpt",
    "MixtralConfig": "mixtral", "MixtralModel": "mixtral",
    "BertConfig": "bert", "BertModel": "bert",
    "T5Config": "t5", "T5Model": "t5",
    "generate": "generation", "sample_logits": "generation",
}


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    return getattr(importlib.import_module(f"{__name__}.{mod}"), name)


__all__ = sorted(_LAZY)
