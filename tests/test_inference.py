"""TransformerInferenceModule on CPU: logits, cached vs uncached generation, checkpoint round trip, recorder."""

from pathlib import Path

import torch
import yaml

from scaling_b200.core.nn.parallel_module.inference_module import RecorderSetting
from scaling_b200.transformer.context.config import TransformerArchitectureConfig
from scaling_b200.transformer.inference import TransformerInferenceModule, sample_argmax
from scaling_b200.transformer.model.model import get_transformer_layer_specs
from scaling_b200.transformer.tokenizer import Tokenizer

ARCH = {"vocab_size": 32, "hidden_size": 32, "num_layers": 2, "num_attention_heads": 4, "sequence_length": 64,
        "precision": "float32", "masked_softmax": {"kernel": "torch"}, "weight_tying": False,
        "relative_position_embedding_type": "rotary"}


def _module(tokenizer=None) -> TransformerInferenceModule:
    torch.manual_seed(0)
    arch = TransformerArchitectureConfig.from_dict(dict(ARCH))
    return TransformerInferenceModule(get_transformer_layer_specs(architecture_config=arch), devices=("cpu",),
                                      tokenizer=tokenizer)


def test_logits_and_generate_cache_agrees_with_recompute():
    m = _module()
    prompt = [3, 7, 1, 9, 4]
    logits = m.logits(input_tokens=prompt)
    assert logits.shape == (5, 32) and torch.isfinite(logits).all()
    cached = m.generate(max_tokens=6, input_tokens=prompt, stop_tokens=[31], use_cache=True)
    plain = m.generate(max_tokens=6, input_tokens=prompt, stop_tokens=[31], use_cache=False)
    assert cached.completion_tokens == plain.completion_tokens
    assert len(cached.completion_tokens) <= 6
    assert cached.completion_logits.shape == (len(cached.completion_tokens), 32)
    assert torch.allclose(cached.completion_logits, plain.completion_logits, atol=1e-4)
    # greedy decoding follows the argmax of the returned logits
    assert cached.completion_tokens == cached.completion_logits.argmax(-1).tolist()


def test_generate_stops_at_stop_token_and_decodes_text():
    tok = Tokenizer.from_words([f"w{i}" for i in range(30)])
    m = _module(tok)
    first = m.generate(max_tokens=1, input_text="w1 w2 w3").completion_tokens[0]
    out = m.generate(max_tokens=8, input_text="w1 w2 w3", stop_tokens=[first])
    assert out.completion_tokens == [first]
    assert isinstance(out.completion_text, str)
    assert sample_argmax(torch.zeros(1, 2, 4)).shape == (1,)


def test_hidden_state_recorder():
    m = _module()
    logits, record = m.logits_with_hidden_state_recorder(input_tokens=[1, 2, 3],
                                                         recorder_settings_per_layer={1: RecorderSetting()})
    assert logits.shape == (3, 32)
    assert list(record.keys()) == [1] and len(record[1]) > 0


def test_from_checkpoint_round_trip(tmp_path: Path):
    m = _module()
    m.save_checkpoint(tmp_path) if hasattr(m, "save_checkpoint") else None
    tok = Tokenizer.from_words([f"w{i}" for i in range(30)])
    (tmp_path / "vocab.json").write_text(tok.tokenizer.to_str())
    (tmp_path / "config.yml").write_text(yaml.safe_dump({"transformer_architecture": dict(ARCH)}))
    if not any(tmp_path.glob("model_state_layer_*")):
        import pytest

        pytest.skip("inference modules cannot write checkpoints")
    loaded = TransformerInferenceModule.from_checkpoint(tmp_path, devices=("cpu",))
    a, b = m.logits(input_tokens=[5, 6, 7]), loaded.logits(input_tokens=[5, 6, 7])
    assert torch.allclose(a, b, atol=1e-6)
    assert loaded.tokenizer is not None


def test_attention_manipulation_controls():
    """Per-token attention controls: factor 1 leaves the logits alone, factor 0 removes the token from every later
    position's view (the positions before it are untouched under the causal mask), both in the log-additive and in
    the multiplicative form."""
    from scaling_b200.transformer.data.inference_settings import (Control, InferenceSettings,
                                                                  InferenceSuppressionParameters)
    from scaling_b200.transformer.data.text_dataset import TextDatasetBatch

    m = _module()
    prompt = [3, 7, 1, 9, 4, 11]

    def run(controls, log_additive=True):
        params = None if controls is None else [InferenceSuppressionParameters(None, log_additive, controls)]
        settings = InferenceSettings(use_cache=False, reset_cache=True, cache_index=0, embedding_layers=[-1],
                                     inference_control_parameters=params)
        batch = TextDatasetBatch(input_token_ids=torch.tensor([prompt]), inference_settings=settings)
        with torch.no_grad():
            return m.forward(batch).activations.squeeze(0)

    plain = run(None)
    assert torch.allclose(run([Control(token_index=2, factor=1.0)]), plain, atol=1e-5)
    assert torch.allclose(run([Control(token_index=2, factor=1.0)], log_additive=False), plain, atol=1e-5)
    for log_additive in (True, False):
        suppressed = run([Control(token_index=2, factor=0.0)], log_additive=log_additive)
        assert torch.allclose(suppressed[:2], plain[:2], atol=1e-5)  # earlier positions never saw token 2
        assert not torch.allclose(suppressed[3:], plain[3:], atol=1e-4)
    damped = run([Control(token_index=2, factor=0.5)])
    gap = lambda t: (t[3:] - plain[3:]).abs().max().item()  # noqa: E731
    assert 0 < gap(damped) < gap(run([Control(token_index=2, factor=0.0)]))


def test_checkpoint_of_a_tensor_parallel_run_loads_into_the_inference_module(tmp_path: Path):
    """Training checkpoints are layout independent: one written by two tensor-parallel ranks (multi-query attention with
    replicated KV projections) gives the logits of the checkpoint written by a single process."""
    import pytest

    from tests.test_finetuning import _embedding_setup
    from tests.test_transformer_training import LLAMA_ARCH, losses

    vocab, _ = _embedding_setup(tmp_path)
    arch = dict(LLAMA_ARCH, attention_num_kv_heads=1, vocab_file=vocab)
    init = str(tmp_path / "init")
    losses(1, save_initial=init, arch=arch, iters=1)
    logits = {}
    for name, ws, kw in (("one", 1, {}), ("tp", 2, dict(mp=2, sp=True))):
        losses(ws, load_dir=init, arch=arch, iters=3, save_dir=str(tmp_path / name), save_interval=3, **kw)
        module = TransformerInferenceModule.from_checkpoint(tmp_path / name / "global_step3", devices=("cpu",))
        logits[name] = module.logits(input_tokens=[3, 9, 27, 81, 5])
    assert logits["one"].shape == (5, 128)
    assert torch.allclose(logits["tp"], logits["one"], atol=2e-4), (logits["tp"] - logits["one"]).abs().max()
    with pytest.raises(AssertionError, match="Config file not found"):
        TransformerInferenceModule.from_checkpoint(tmp_path / "one", devices=("cpu",))  # the step folder is the checkpoint


def test_sentence_embeddings_from_a_model_without_a_language_model_head():
    """``encode`` returns one row of hidden states per sentence, padded to the longest prompt of its batch; an
    instruction lengthens every prompt, ``max_length`` cuts it."""
    tok = Tokenizer.from_words([f"w{i}" for i in range(30)])
    torch.manual_seed(0)
    arch = TransformerArchitectureConfig.from_dict(dict(ARCH, lm_head=False))
    m = TransformerInferenceModule(get_transformer_layer_specs(architecture_config=arch), devices=("cpu",),
                                   tokenizer=tok)
    marks = dict(user_token="w1 ", embed_token="w2 ", pad_token="w0")
    two = m.encode(["w5 w6", "w7 w8 w9 w10"], **marks)
    one = m.encode("w5 w6 w7 w8 w9 w10", convert_to_tensor=True, **marks)
    assert two.shape == (2, 6, 32) and tuple(one.shape) == (1, 8, 32) and isinstance(one, torch.Tensor)
    assert torch.isfinite(torch.as_tensor(two)).all()
    instructed = m.encode(["w5 w6"] * 5, instruction="w11 w12 ", batch_size=2, **marks)
    assert instructed.shape == (5, 6, 32)
    assert m.encode(["w5 " * 40], max_length=16, **marks).shape == (1, 16, 32)
    assert m.encode_queries(["w5 w6"], **marks).shape == m.encode_corpus([{"title": "w5", "text": "w6"}], **marks).shape
