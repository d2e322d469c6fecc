"""Oracle-internal consistency of the two model loops (CPU only): decode_next after a prefill
must continue exactly where a longer prefill would be, and error statuses follow the reference."""
import numpy as np
import pytest

from zignn_b200 import ggml, hostmodel

GPT2_TINY = dict(vocab=300, embed=64, head=4, layer=2, ctx=32, ffn=128)
GEMMA_TINY = dict(vocab=512, embed=64, head=4, head_kv=1, head_dim=32, layer=6, ctx=48, ffn=128,
                  rope_base=1000000.0, sliding_window=8, rms_eps=1e-6, global_every=6)


def rel_l2(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def test_gpt2_prefill_then_decode_equals_longer_prefill(oracle):
    host = hostmodel.Gpt2Host.synthetic(GPT2_TINY, seed=1, std=0.08).randomize_small_params()
    toks = np.random.default_rng(0).integers(0, 300, size=12)
    m1 = oracle.Gpt2(host, 2)
    m1.prefill(toks[:8])
    for t in toks[8:11]:
        m1.decode_next(t)
    a = m1.decode_next(toks[11])
    m2 = oracle.Gpt2(host, 1)
    b = m2.prefill(toks)
    assert rel_l2(a, b) < 1e-5


def test_gemma3_prefill_then_decode_equals_longer_prefill(oracle):
    host = hostmodel.Gemma3Host.synthetic(GEMMA_TINY, qtype=ggml.Q4_0, embd_qtype=ggml.Q8_0,
                                          down_qtype=ggml.Q4_1, seed=1, std=0.08).randomize_small_params()
    toks = np.random.default_rng(0).integers(0, 512, size=20)  # longer than the window of 8
    m1 = oracle.Gemma3(host, 2)
    m1.prefill(toks[:15])
    for t in toks[15:19]:
        m1.decode_next(t)
    a = m1.decode_next(toks[19])
    m2 = oracle.Gemma3(host, 3)
    b = m2.prefill(toks)
    assert rel_l2(a, b) < 1e-5


def test_sequence_errors(oracle):
    host = hostmodel.Gpt2Host.synthetic(GPT2_TINY, seed=1)
    m = oracle.Gpt2(host, 1)
    with pytest.raises(RuntimeError):
        m.prefill([])  # error.EmptySequence
    with pytest.raises(RuntimeError):
        m.prefill(np.zeros(33, np.uint32))  # error.SequenceTooLong
    m.prefill(np.zeros(32, np.uint32))
    with pytest.raises(RuntimeError):
        m.decode_next(0)  # error.ContextFull
