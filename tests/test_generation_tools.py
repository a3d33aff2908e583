"""Sampling, chat engine, checkpoint loading for the tools, layer streaming, data monitor (all CPU)."""
import copy
import json
import types

import torch

from maester_b200.chat import (ChatMLFormatter, ChatSession, GenerationConfig, LayerStreamingRunner, Message,
                               PlainFormatter, RawFormatter, load_model_from_dcp)
from maester_b200.convert.io import write_dcp
from maester_b200.data_monitor import DataMonitor, find_tokenizer
from maester_b200.generate import generate, greedy, logits_to_probs, multinomial_sample_one_no_sync, sample
from maester_b200.models import model_name_to_cls, models_config


class CharTokenizer:
    eos_token_id = 0

    def encode(self, s):
        return [min(ord(c), 127) for c in s]

    def decode(self, ids):
        return "".join(chr(i) if 32 <= i < 127 else "?" for i in ids)


def _tiny_llama(vocab=128):
    a = copy.deepcopy(models_config["llama3"]["tiny"])
    a.vocab_size, a.max_seq_len = vocab, 128
    torch.manual_seed(0)
    return a, model_name_to_cls["llama3"].from_model_args(a).eval()


def test_sampling_primitives():
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0]])
    p = logits_to_probs(logits, temperature=1.0, top_k=2)
    assert p[0, :2].sum() == 0 and abs(p.sum().item() - 1) < 1e-6
    tok, _ = sample(logits, temperature=0.0)
    assert tok.item() == 3
    g = torch.Generator().manual_seed(0)
    draws = torch.cat([multinomial_sample_one_no_sync(torch.tensor([[0.1, 0.9]]), g) for _ in range(400)])
    assert 0.8 < draws.float().mean().item() < 0.97


def test_generate_greedy_is_argmax_rollout():
    _, m = _tiny_llama()
    prompt = torch.randint(1, 128, (2, 5))
    out = greedy(m, prompt, 4)
    assert out.shape == (2, 9) and torch.equal(out[:, :5], prompt)
    with torch.no_grad():
        assert torch.equal(out[:, 5], m(prompt)[:, -1].argmax(-1))
    seen = []
    generate(m, prompt, 3, temperature=1.0, top_k=5, callback=seen.append)
    assert len(seen) == 3 and seen[0].shape == (2, 1)


def test_formatters():
    h = [Message("user", "hi"), Message("assistant", "yo"), Message("user", "bye")]
    s = ChatMLFormatter(system="be brief").render(h)
    assert s.startswith("<|im_start|>system\nbe brief<|im_end|>\n") and s.endswith("<|im_start|>assistant\n")
    assert PlainFormatter().render(h).endswith("User: bye\nAssistant:")
    assert RawFormatter().render(h) == "hiyobye"


def test_chat_session_streams_and_keeps_history():
    _, m = _tiny_llama()
    sess = ChatSession(m, CharTokenizer(), PlainFormatter(), GenerationConfig(max_new_tokens=6, temperature=0.0, top_k=None, window=64))
    pieces = list(sess.stream("hello"))
    assert [x.role for x in sess.history] == ["user", "assistant"]
    assert "".join(pieces) == sess.history[-1].content and len(sess.history[-1].content) <= 6


def test_load_model_from_dcp_matches_source(tmp_path):
    a, m = _tiny_llama(vocab=96)
    ck = tmp_path / "job" / "checkpoints" / "step-3"
    write_dcp(ck, {k: v.detach() for k, v in m.state_dict().items()})
    (tmp_path / "job" / "config.json").write_text(json.dumps({"model_name": "llama3", "flavor": "tiny", "seq_len": 128}))
    loaded, args = load_model_from_dcp(str(ck))
    assert args.vocab_size == 96
    tok = torch.randint(0, 96, (1, 12))
    with torch.no_grad():
        assert torch.allclose(loaded(tok), m(tok), atol=1e-5)


def test_layer_streaming_equals_plain_forward():
    a = copy.deepcopy(models_config["glm4"]["debug"])
    a.vocab_size = 256
    torch.manual_seed(1)
    m = model_name_to_cls["glm4"].from_model_args(a).eval()
    m.init_weights()
    tok = torch.randint(0, 256, (1, 16))
    with torch.no_grad():
        want = m(tok)
        got = LayerStreamingRunner(m, torch.device("cpu"), block=1)(tok)
    assert torch.allclose(got, want, atol=1e-5)


def test_data_monitor_reports():
    _, m = _tiny_llama()
    state = types.SimpleNamespace(step=100)
    inner = types.SimpleNamespace(tokenizer=CharTokenizer())
    chain = types.SimpleNamespace(dataset=types.SimpleNamespace(data=[inner]))
    assert find_tokenizer(chain) is inner.tokenizer
    mon = DataMonitor(state, log_freq=50, sample_size=1, top_k=3, prompts=["ab"])
    ids = torch.randint(33, 120, (2, 24))
    labels = torch.cat([ids[:, 1:], torch.full((2, 1), -100)], dim=1)
    txt = mon.log_batch_samples(ids, labels, chain)
    assert "shifted by one: True" in txt and "masked label positions: 1" in txt
    with torch.no_grad():
        pred = m(ids)
    assert "top-3 predictions" in mon.log_predictions(pred, labels, chain, context=ids)
    gen = mon.log_generations(m, ids, chain, max_tokens=3, prefix_len=4)
    assert "prompt 'ab'" in gen and "batch prefix" in gen
    state.step = 101
    assert mon.log_batch_samples(ids, labels, chain) is None
    assert "dataset chain" in mon.log_dataset_stats(chain)
