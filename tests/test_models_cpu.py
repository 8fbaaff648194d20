"""Model families against the Hugging Face implementations of the same architectures (random weights, fp32, CPU):
a converted checkpoint must give the same logits, decoding on the key/value cache must give the tokens of a full
recompute, and the conversion must round-trip.  (Test model: the accuracy checks of the reference's
``docs/examples/te_llama`` / ``te_gemma`` tutorials, which compare against the Hugging Face model.)"""
import os
import socket
import warnings

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from transformerengine_b200.models import hf
from transformerengine_b200.models.generation import generate, sample_logits

transformers = pytest.importorskip("transformers")

BASE = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=64, attn_implementation="eager")


def _hf_model(family):
    T = transformers
    if family == "llama":
        return T.LlamaForCausalLM(T.LlamaConfig(**BASE, rms_norm_eps=1e-5, rope_theta=10000.0,
                                                tie_word_embeddings=False))
    if family == "llama_tied":
        return T.LlamaForCausalLM(T.LlamaConfig(**BASE, rms_norm_eps=1e-5, tie_word_embeddings=True))
    if family == "mistral":
        return T.MistralForCausalLM(T.MistralConfig(**BASE, sliding_window=4, rms_norm_eps=1e-5))
    if family == "gemma":
        return T.GemmaForCausalLM(T.GemmaConfig(**BASE, head_dim=32, rms_norm_eps=1e-6))
    if family == "qwen3":
        return T.Qwen3ForCausalLM(T.Qwen3Config(**BASE, head_dim=24, rms_norm_eps=1e-6, tie_word_embeddings=False))
    if family == "mixtral":
        return T.MixtralForCausalLM(T.MixtralConfig(**BASE, num_local_experts=4, num_experts_per_tok=2,
                                                    rms_norm_eps=1e-5))
    raise ValueError(family)


CONVERT = {"llama": hf.llama_from_hf, "llama_tied": hf.llama_from_hf, "mistral": hf.mistral_from_hf,
           "gemma": hf.gemma_from_hf, "qwen3": hf.qwen3_from_hf, "mixtral": hf.mixtral_from_hf}


def _randomize(m):
    """Norm weights start at their identity value and routers / experts at zero-ish scales: perturb them so that
    a wrong mapping cannot hide."""
    with torch.no_grad():
        for k, p in m.named_parameters():
            if "norm" in k:
                p.add_(torch.randn_like(p) * 0.1)
            elif "experts" in k or k.endswith("gate.weight"):
                p.normal_(0, 0.05)


def _greedy_by_recompute(model, tokens, n):
    ref = tokens.clone()
    with torch.no_grad():
        for _ in range(n):
            logits = model(ref)              # [s, b, vocab]
            ref = torch.cat([ref, logits[-1].argmax(-1)[:, None]], 1)
    return ref


@pytest.mark.parametrize("family", list(CONVERT))
def test_converted_checkpoint_matches_hugging_face(family):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ref = _hf_model(family).eval()
    _randomize(ref)
    kw = dict(pad_align=8) if family == "mixtral" else {}
    ours = CONVERT[family](ref, device="cpu", params_dtype=torch.float32, **kw).eval()
    tokens = torch.randint(0, 128, (2, 12))
    with torch.no_grad():
        want = ref(tokens).logits
        got = ours(tokens).transpose(0, 1)
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    # decoding on the cache (prefill + one token per step) reproduces a full recompute per token
    assert torch.equal(ours.generate(tokens, 4), _greedy_by_recompute(ours, tokens, 4))
    if family != "mixtral":
        back = hf.export_hf_llama_state_dict(ours)
        for k, v in ref.state_dict().items():
            assert torch.equal(back[k], v), k


def test_tied_head_is_one_parameter():
    from transformerengine_b200.models.gemma import GemmaConfig, GemmaModel
    m = GemmaModel(GemmaConfig.tiny(params_dtype=torch.float32), device="cpu")
    assert m.lm_head.weight is m.embedding.weight
    n = sum(p.numel() for p in m.parameters())
    assert n == m.cfg.num_params(), (n, m.cfg.num_params())
    loss = m(torch.randint(0, 512, (2, 8)), labels=torch.randint(0, 512, (2, 8)))
    loss.backward()
    assert m.embedding.weight.grad is not None and torch.isfinite(m.embedding.weight.grad).all()


@pytest.mark.parametrize("family", ["mistral", "qwen3", "gemma"])
def test_family_trains(family):
    from transformerengine_b200.models.gemma import GemmaConfig, GemmaModel
    from transformerengine_b200.models.mistral import MistralConfig, MistralModel
    from transformerengine_b200.models.qwen import Qwen3Config, Qwen3Model
    cfg_cls, cls = {"mistral": (MistralConfig, MistralModel), "qwen3": (Qwen3Config, Qwen3Model),
                    "gemma": (GemmaConfig, GemmaModel)}[family]
    m = cls(cfg_cls.tiny(params_dtype=torch.float32), device="cpu")
    assert sum(p.numel() for p in m.parameters()) == m.cfg.num_params()
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    tokens = torch.randint(0, 512, (2, 16))
    losses = []
    for _ in range(8):
        loss = m(tokens, labels=tokens)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.5, losses


def test_generation_with_ragged_prompts_paged_cache_and_eos():
    from transformerengine_b200.models.llama import LlamaConfig, LlamaModel
    m = LlamaModel(LlamaConfig.tiny(params_dtype=torch.float32), device="cpu").eval()
    prompt = torch.randint(1, 1024, (3, 6))
    lens = torch.tensor([6, 3, 4])
    out = m.generate(prompt, 4, prompt_lengths=lens, is_paged=True, page_size=4, total_num_pages=12)
    assert out.shape == (3, 10)
    for i, n in enumerate(lens.tolist()):
        want = _greedy_by_recompute(m, prompt[i:i + 1, :n], 4)[0]
        assert torch.equal(out[i, :n + 4], want), i
        assert (out[i, n + 4:] == 0).all()
    # a sequence that emits the stop token leaves the batch; the others go on
    first = int(_greedy_by_recompute(m, prompt[1:2, :3], 1)[0, -1])
    out2 = m.generate(prompt, 4, prompt_lengths=lens, eos_token_id=first, pad_token_id=0)
    assert out2[1, 3] == first and (out2[1, 4:] == 0).all()
    for i in (0, 2):
        want = _greedy_by_recompute(m, prompt[i:i + 1, :lens[i]], 4)[0]
        stop = (want[lens[i]:] == first).nonzero()
        upto = lens[i] + (int(stop[0]) + 1 if len(stop) else 4)
        assert torch.equal(out2[i, :upto], want[:upto])


def test_sampling_filters():
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0, 4.0]]).log_softmax(-1).repeat(64, 1)
    g = torch.Generator().manual_seed(0)
    assert (sample_logits(logits) == 4).all()
    assert set(sample_logits(logits, 1.0, top_k=2, generator=g).tolist()) <= {3, 4}
    # nucleus: p(4) = 0.636, p(3) = 0.234 -> top_p 0.7 keeps exactly those two
    assert set(sample_logits(logits, 1.0, top_p=0.7, generator=g).tolist()) == {3, 4}
    assert set(sample_logits(logits, 1.0, top_p=0.5, generator=g).tolist()) == {4}
    assert len(set(sample_logits(logits, 5.0, generator=g).tolist())) >= 4
    assert generate.__doc__


# ------------------------------------------------------------------ tensor-parallel shards of a checkpoint
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _tp_worker(rank, world, port, sd, tokens, q, family="llama"):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from transformerengine_b200.models.gemma import GemmaConfig, GemmaModel
        from transformerengine_b200.models.llama import LlamaConfig, LlamaModel
        base = dict(vocab_size=128, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=128,
                    rope_theta=10000.0, params_dtype=torch.float32)
        if family == "gpt2":
            from transformerengine_b200.models.gpt import GPTConfig, GPTModel, load_hf_gpt2
            m = GPTModel(GPTConfig(vocab_size=128, max_positions=64, hidden_size=64, num_layers=2, num_heads=4,
                                   params_dtype=torch.float32), tp_group=dist.group.WORLD, device="cpu").eval()
            load_hf_gpt2(m, sd)
            with torch.no_grad():
                logits = m(tokens)
            parts = [torch.empty_like(logits) for _ in range(world)]
            dist.all_gather(parts, logits)
            if rank == 0:
                q.put(torch.cat(parts, dim=-1))
            return
        if family == "gemma":
            m = GemmaModel(GemmaConfig(**base, head_dim=32, rms_eps=1e-6), tp_group=dist.group.WORLD, device="cpu").eval()
            assert m.lm_head.weight is m.embedding.weight and m.embedding.weight.shape == (64, 64)
        else:
            m = LlamaModel(LlamaConfig(**base), tp_group=dist.group.WORLD, device="cpu").eval()
        hf.load_hf_llama(m, sd)
        with torch.no_grad():
            logits = m(tokens)                         # [s, b, vocab / tp]
        parts = [torch.empty_like(logits) for _ in range(world)]
        dist.all_gather(parts, logits)
        if rank == 0:
            q.put(torch.cat(parts, dim=-1))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("family", ["llama", "gemma", "gpt2"])
def test_checkpoint_loads_into_tensor_parallel_shards(family):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        if family == "gpt2":
            T = transformers
            ref = T.GPT2LMHeadModel(T.GPT2Config(vocab_size=128, n_positions=64, n_embd=64, n_layer=2, n_head=4,
                                                 attn_implementation="eager", resid_pdrop=0.0, embd_pdrop=0.0,
                                                 attn_pdrop=0.0)).eval()
            _perturb(ref, ("ln_", "bias"))
        else:
            ref = _hf_model(family).eval()
    _randomize(ref)
    tokens = torch.randint(0, 128, (2, 8))
    with torch.no_grad():
        want = ref(tokens).logits
    sd = {k: v.clone() for k, v in ref.state_dict().items()}
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, sd, tokens, q, family)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert torch.allclose(got.transpose(0, 1), want, atol=2e-5), float((got.transpose(0, 1) - want).abs().max())


# ------------------------------------------------------------------ GPT-2, BERT, T5
def _perturb(m, names):
    with torch.no_grad():
        for k, p in m.named_parameters():
            if any(n in k for n in names):
                p.add_(torch.randn_like(p) * 0.1)


def test_gpt2_checkpoint_matches_hugging_face():
    from transformerengine_b200.models.gpt import gpt_from_hf
    T = transformers
    ref = T.GPT2LMHeadModel(T.GPT2Config(vocab_size=128, n_positions=64, n_embd=64, n_layer=2, n_head=4,
                                         attn_implementation="eager", resid_pdrop=0.0, embd_pdrop=0.0,
                                         attn_pdrop=0.0)).eval()
    _perturb(ref, ("ln_", "bias"))
    ours = gpt_from_hf(ref, device="cpu", params_dtype=torch.float32).eval()
    assert ours.lm_head.weight is ours.embedding.weight
    assert sum(p.numel() for p in ours.parameters()) == ours.cfg.num_params()
    tokens = torch.randint(0, 128, (2, 12))
    with torch.no_grad():
        want = ref(tokens).logits
        got = ours(tokens).transpose(0, 1)
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    assert torch.equal(ours.generate(tokens, 4), _greedy_by_recompute(ours, tokens, 4))
    loss = ours.train()(tokens, labels=tokens)
    want_loss = ref(tokens, labels=tokens).loss
    # the library's loss averages over all b * s rows (the last position has no target and counts as ignored)
    assert torch.allclose(loss, want_loss, atol=1e-4), (float(loss), float(want_loss))


def test_bert_checkpoint_matches_hugging_face():
    from transformerengine_b200.models.bert import bert_from_hf
    T = transformers
    ref = T.BertForMaskedLM(T.BertConfig(vocab_size=128, max_position_embeddings=64, hidden_size=64,
                                         num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                                         hidden_act="gelu_pytorch_tanh", attn_implementation="eager",
                                         hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)).eval()
    _perturb(ref, ("LayerNorm", "bias"))
    ours = bert_from_hf(ref, device="cpu", params_dtype=torch.float32).eval()
    tokens = torch.randint(0, 128, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[1, 8:] = 0
    segments = torch.randint(0, 2, (2, 12))
    with torch.no_grad():
        want = ref(tokens, attention_mask=mask, token_type_ids=segments).logits
        got = ours(tokens, mask, segments).transpose(0, 1)
    assert torch.isfinite(got).all()
    assert torch.allclose(got[mask.bool()], want[mask.bool()], atol=2e-5)
    labels = tokens.clone()
    labels[mask == 0] = -100
    loss = ours.train()(tokens, mask, segments, labels=labels)
    loss.backward()
    want_loss = ref(tokens, attention_mask=mask, token_type_ids=segments, labels=labels).loss
    assert torch.allclose(loss, want_loss, atol=1e-4)
    assert ours.word_embeddings.weight.grad is not None


@pytest.mark.parametrize("mlp,tied", [("gated-gelu", False), ("relu", True)])
def test_t5_checkpoint_matches_hugging_face(mlp, tied):
    from transformerengine_b200.models.t5 import t5_from_hf
    T = transformers
    ref = T.T5ForConditionalGeneration(T.T5Config(
        vocab_size=128, d_model=64, d_kv=24, d_ff=128, num_layers=2, num_decoder_layers=2, num_heads=4,
        relative_attention_num_buckets=8, relative_attention_max_distance=16, feed_forward_proj=mlp,
        tie_word_embeddings=tied, dropout_rate=0.0, decoder_start_token_id=0, attn_implementation="eager")).eval()
    with torch.no_grad():
        for k, p in ref.named_parameters():
            if "layer_norm" in k:
                p.add_(torch.randn_like(p) * 0.1)
            elif "relative" in k:
                p.normal_(0, 0.5)
            elif k == "shared.weight":
                p.mul_(0.3)
    ours = t5_from_hf(ref, device="cpu", params_dtype=torch.float32).eval()
    assert ours.cfg.scale_decoder_outputs == tied
    tokens, dec = torch.randint(1, 128, (2, 20)), torch.randint(1, 128, (2, 9))
    mask = torch.ones(2, 20, dtype=torch.long)
    mask[1, 13:] = 0
    with torch.no_grad():
        want = ref(input_ids=tokens, attention_mask=mask, decoder_input_ids=dec).logits
        got = ours(tokens, mask, decoder_tokens=dec).transpose(0, 1)
    assert torch.allclose(got, want, atol=5e-5, rtol=1e-5), float((got - want).abs().max())
    labels = torch.randint(1, 128, (2, 9))
    labels[0, 6:] = -100
    loss = ours.train()(tokens, mask, labels=labels)
    loss.backward()
    want_loss = ref(input_ids=tokens, attention_mask=mask, labels=labels).loss
    assert torch.allclose(loss, want_loss, atol=1e-4), (float(loss), float(want_loss))
    # greedy decoding: first tokens agree with the reference implementation's own loop
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        theirs = ref.generate(input_ids=tokens, attention_mask=mask, max_new_tokens=3, do_sample=False)
    mine = ours.generate(tokens, 3, mask)
    assert torch.equal(mine[:, :2], theirs[:, :2])


def test_relative_position_buckets():
    from transformerengine_b200.models.t5 import relative_position_bucket
    rel = torch.arange(-40, 41)
    uni = relative_position_bucket(rel, False, 8, 16)
    assert uni[rel >= 0].eq(0).all()                       # a causal stack never looks ahead
    assert uni[rel == -1] == 1 and uni[rel == -3] == 3     # exact buckets for small offsets
    assert uni[rel <= -16].eq(7).all()                     # one bucket beyond max_distance
    assert (uni[:-1] >= uni[1:]).all()                     # monotone in the distance
    bi = relative_position_bucket(rel, True, 8, 16)
    assert bi[rel < 0].max() < 4 <= bi[rel > 0].min()      # half of the buckets per direction


def test_layers_inside_a_hugging_face_pretrained_model(tmp_path):
    """A ``transformers.PreTrainedModel`` that contains this library's layers saves (safetensors) and loads back
    (test model: the reference's ``tests/pytorch/test_hf_integration.py``)."""
    import transformerengine_b200 as te
    from transformers.configuration_utils import PretrainedConfig
    from transformers.modeling_utils import PreTrainedModel

    class SimpleModel(PreTrainedModel):
        config_class = PretrainedConfig

        def __init__(self, config):
            super().__init__(config)
            self.my_layer = te.TransformerLayer(hidden_size=64, num_attention_heads=4, ffn_hidden_size=128,
                                                layer_number=None, device="cpu", params_dtype=torch.float32,
                                                hidden_dropout=0.0, attention_dropout=0.0)
            self.post_init()

        def forward(self, hidden_states, attention_mask=None):
            return self.my_layer(hidden_states, attention_mask)

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        model = SimpleModel(PretrainedConfig()).eval()
        model.save_pretrained(tmp_path / "simple_model")
        again = SimpleModel.from_pretrained(tmp_path / "simple_model").eval()
    x = torch.randn(8, 2, 64)
    assert torch.equal(model(x), again(x))
