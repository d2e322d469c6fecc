"""Decode engines against the oracle's model loops: logits within rel-L2 1e-3 and identical greedy
tokens for the first 64 steps (the stated bar), on small and on full-size configurations."""
import numpy as np
import pytest
import torch

from zignn_b200 import ggml, hostmodel

pytestmark = pytest.mark.gpu

GPT2_TINY = dict(vocab=1000, embed=128, head=4, layer=2, ctx=96, ffn=512)
GEMMA_TINY = dict(vocab=2048, embed=128, head=4, head_kv=1, head_dim=32, layer=7, ctx=96, ffn=256,
                  rope_base=1000000.0, sliding_window=16, rms_eps=1e-6, global_every=6)


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def run_parity(zq_engine, oracle_model, prompt, n_steps):
    """Greedy decoding on both sides; returns (gpu tokens, cpu tokens, logits rel-L2 of every step
    while the token streams agree)."""
    lg = zq_engine.prefill(prompt).cpu().numpy()
    lc = oracle_model.prefill(prompt)
    errs = [rel_l2(lg, lc)]
    gt, ct = [], []
    for _ in range(n_steps):
        tg, tc = int(np.argmax(lg)), int(np.argmax(lc))
        gt.append(tg)
        ct.append(tc)
        if tg != tc:
            break
        lg = zq_engine.decode_next(tg).cpu().numpy()
        lc = oracle_model.decode_next(tc)
        errs.append(rel_l2(lg, lc))
    return gt, ct, errs


def test_gpt2_tiny_parity(zq, oracle):
    host = hostmodel.Gpt2Host.synthetic(GPT2_TINY, seed=42, std=0.08).randomize_small_params()
    prompt = np.random.default_rng(44).integers(0, GPT2_TINY["vocab"], size=20)
    gt, ct, errs = run_parity(zq.Gpt2(host), oracle.Gpt2(host, 4), prompt, 64)
    assert gt == ct
    assert max(errs) <= 1e-5, max(errs)  # f32 activations: no quantiser in the loop


@pytest.mark.parametrize("qtypes", [(ggml.Q8_0, ggml.Q8_0, ggml.Q8_0), (ggml.Q4_0, ggml.Q8_0, ggml.Q4_1),
                                    (ggml.Q4_1, ggml.Q4_1, ggml.Q4_1)])
def test_gemma3_tiny_parity(zq, oracle, qtypes):
    q, embd, down = qtypes
    host = hostmodel.Gemma3Host.synthetic(GEMMA_TINY, qtype=q, embd_qtype=embd, down_qtype=down, seed=42,
                                          std=0.08).randomize_small_params()
    prompt = np.random.default_rng(44).integers(0, GEMMA_TINY["vocab"], size=24)  # beyond the window of 16
    gt, ct, errs = run_parity(zq.Gemma3(host), oracle.Gemma3(host, 4), prompt, 64)
    assert gt == ct
    # Every op of this path is evaluated in the CPU code's order, so the logits are the same bits.
    # (The Q8 activation quantiser makes anything less than that chaotic: one activation that differs
    # in its last bit can round to the other integer and move the logits of a 128-wide model by 1e-2.)
    assert max(errs) == 0.0, errs


def test_gemma3_batched_sequences_bit_exact(zq, oracle):
    """Seven independent sequences with different prompt lengths decoded together: each sequence's logits
    must be the bits of decoding it alone on the CPU path (the linears run as exact int8 GEMMs over the
    sequences; positions, windows and cache slots are per sequence)."""
    host = hostmodel.Gemma3Host.synthetic(GEMMA_TINY, qtype=ggml.Q8_0, seed=7, std=0.08).randomize_small_params()
    n_seq, steps = 7, 12
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, GEMMA_TINY["vocab"], size=int(n)) for n in (1, 3, 9, 17, 20, 24, 30)]
    eng = zq.Gemma3Batch(host, n_seq)
    refs = [oracle.Gemma3(host, 2) for _ in range(n_seq)]
    toks = []
    for i, p in enumerate(prompts):
        lg = eng.prefill(i, p).cpu().numpy()
        lc = refs[i].prefill(p)
        assert np.array_equal(lg, lc), "prefill of sequence %d" % i
        toks.append(int(np.argmax(lc)))
        assert eng.seq_len(i) == len(p)
    for s in range(steps):
        lg = eng.decode_next(toks).cpu().numpy()
        for i in range(n_seq):
            lc = refs[i].decode_next(toks[i])
            assert np.array_equal(lg[i], lc), "step %d sequence %d" % (s, i)
            toks[i] = int(np.argmax(lc))
    assert [eng.seq_len(i) for i in range(n_seq)] == [len(p) + steps for p in prompts]


def test_device_greedy_loop_matches_stepwise(zq):
    host = hostmodel.Gemma3Host.synthetic(GEMMA_TINY, qtype=ggml.Q8_0, seed=3, std=0.08)
    prompt = np.random.default_rng(1).integers(0, GEMMA_TINY["vocab"], size=8)
    a, b = zq.Gemma3(host), zq.Gemma3(host)
    first = int(a.prefill(prompt).argmax().item())
    b.prefill(prompt)
    toks = a.decode_greedy(first, 20)
    step, tok = [], first
    for _ in range(20):
        tok = int(b.decode_next(tok).argmax().item())
        step.append(tok)
    assert list(toks) == step
    assert a.seq_len == b.seq_len == 28


def test_sequence_error_statuses(zq):
    from zignn_b200 import _lib
    host = hostmodel.Gpt2Host.synthetic(dict(vocab=64, embed=32, head=2, layer=1, ctx=8, ffn=64), seed=1)
    m = zq.Gpt2(host)
    for bad in ([], np.zeros(9, np.uint32)):
        with pytest.raises(_lib.ZqError) as e:
            m.prefill(bad)
        assert e.value.status == 6  # EmptySequence / SequenceTooLong
    m.prefill(np.zeros(8, np.uint32))
    with pytest.raises(_lib.ZqError) as e:
        m.decode_next(0)
    assert e.value.status == 6  # ContextFull
    m.reset_cache()
    assert m.seq_len == 0
    m.decode_next(3)
    assert m.seq_len == 1


def test_gpt2_small_full_size_greedy_64(zq, oracle):
    """GPT-2 small, Q4_0, seed 42, 32-token prompt, first 64 greedy tokens identical."""
    host = hostmodel.Gpt2Host.synthetic(hostmodel.GPT2_SMALL, qtype=ggml.Q4_0, seed=42, std=0.02, device="cuda")
    prompt = np.random.default_rng(44).integers(0, 50257, size=32)
    gt, ct, errs = run_parity(zq.Gpt2(host), oracle.Gpt2(host, 8), prompt, 64)
    print("gpt2 full-size logits rel-L2: max %.2e median %.2e" % (max(errs), float(np.median(errs))))
    assert gt == ct, (len(gt), gt[-1], ct[-1])
    assert max(errs) <= 1e-3, max(errs)


def test_gemma3_1b_full_size_greedy_64(zq, oracle):
    """Gemma-3-1B shape, Q8_0, seed 42, 16-token prompt, first 64 greedy tokens identical."""
    host = hostmodel.Gemma3Host.synthetic(hostmodel.GEMMA3_1B, qtype=ggml.Q8_0, seed=42, std=0.02, device="cuda")
    prompt = np.random.default_rng(44).integers(0, 262144, size=16)
    gt, ct, errs = run_parity(zq.Gemma3(host), oracle.Gemma3(host, 8), prompt, 64)
    print("gemma3 full-size logits rel-L2: max %.2e median %.2e" % (max(errs), float(np.median(errs))))
    assert gt == ct, (len(gt), gt[-1], ct[-1])
    assert max(errs) <= 1e-3, max(errs)


def test_gemma3_1b_full_size_prefill_across_the_sliding_window(zq, oracle):
    """Gemma-3-1B shape, Q8_0: a 520-token prefill (five chunks through the exact int8 GEMM, the last rows
    beyond the 512-token window of the local layers) and eight greedy steps; logits are the CPU path's bits."""
    import os
    host = hostmodel.Gemma3Host.synthetic(hostmodel.GEMMA3_1B, qtype=ggml.Q8_0, seed=42, std=0.02, device="cuda")
    prompt = np.random.default_rng(45).integers(0, 262144, size=520)
    eng, ref = zq.Gemma3(host), oracle.Gemma3(host, os.cpu_count() or 8)
    lg, lc = eng.prefill(prompt).cpu().numpy(), ref.prefill(prompt)
    assert np.array_equal(lg, lc), rel_l2(lg, lc)
    for step in range(8):
        t = int(np.argmax(lc))
        assert int(np.argmax(lg)) == t
        lg, lc = eng.decode_next(t).cpu().numpy(), ref.decode_next(t)
        assert np.array_equal(lg, lc), (step, rel_l2(lg, lc))
    assert eng.seq_len == 528


def test_gemma3_1b_q4_1_batched_sequences_full_size(zq, oracle):
    """Gemma-3-1B shape with Q4_1 weights, four independent sequences of different lengths (one beyond the
    sliding window) advanced together: each sequence's logits are the bits of decoding it alone on the CPU."""
    import os
    host = hostmodel.Gemma3Host.synthetic(hostmodel.GEMMA3_1B, qtype=ggml.Q4_1, seed=42, std=0.02, device="cuda")
    rng = np.random.default_rng(46)
    prompts = [rng.integers(0, 262144, size=n) for n in (3, 40, 130, 530)]
    eng = zq.Gemma3Batch(host, len(prompts))
    refs = [oracle.Gemma3(host, os.cpu_count() or 8) for _ in prompts]
    toks = []
    for i, p in enumerate(prompts):
        lg, lc = eng.prefill(i, p).cpu().numpy(), refs[i].prefill(p)
        assert np.array_equal(lg, lc), ("prefill", i, rel_l2(lg, lc))
        toks.append(int(np.argmax(lc)))
    for step in range(4):
        lg = eng.decode_next(toks).cpu().numpy()
        for i in range(len(prompts)):
            lc = refs[i].decode_next(toks[i])
            assert np.array_equal(lg[i], lc), (step, i, rel_l2(lg[i], lc))
            toks[i] = int(np.argmax(lc))


def test_reset_cache_restarts_every_sequence_of_a_batch_engine(zq):
    """reset_cache, then the same prefills and steps again: positions restart at zero for every sequence and
    the logits repeat bit for bit; the one-sequence engine keeps its per-sequence length in step."""
    host = hostmodel.Gemma3Host.synthetic(GEMMA_TINY, qtype=ggml.Q8_0, seed=9, std=0.08).randomize_small_params()
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, GEMMA_TINY["vocab"], size=n) for n in (5, 19, 30)]
    eng = zq.Gemma3Batch(host, 3)

    def run():
        out = [eng.prefill(i, p).cpu() for i, p in enumerate(prompts)]
        toks = [int(o.argmax()) for o in out]
        for _ in range(6):
            lg = eng.decode_next(toks).cpu()
            out.append(lg)
            toks = [int(r.argmax()) for r in lg]
        return out

    first = run()
    assert [eng.seq_len(i) for i in range(3)] == [len(p) + 6 for p in prompts]
    eng.reset_cache()
    assert [eng.seq_len(i) for i in range(3)] == [0, 0, 0]
    second = run()
    assert all(torch.equal(a, b) for a, b in zip(first, second))
    one = zq.Gemma3(host)
    t = int(one.prefill(prompts[0]).argmax())
    one.decode_next(t)
    one.decode_greedy(t, 3)
    assert one.seq_len == len(prompts[0]) + 4 == one.seq_len_of(0)


@pytest.mark.parametrize("qtypes", [(ggml.Q8_0, ggml.Q8_0, ggml.Q8_0), (ggml.Q4_0, ggml.Q8_0, ggml.Q4_1),
                                    (ggml.Q4_1, ggml.Q4_1, ggml.Q4_1)])
def test_persistent_decode_kernel_equals_the_launch_sequence(zq, qtypes):
    """One cooperative kernel per token against the captured launch sequence: same logits bit for bit, step
    by step and through the on-device greedy loop (window 16 crossed, global layer included)."""
    q, embd, down = qtypes
    host = hostmodel.Gemma3Host.synthetic(GEMMA_TINY, qtype=q, embd_qtype=embd, down_qtype=down, seed=11,
                                          std=0.08).randomize_small_params()
    prompt = np.random.default_rng(3).integers(0, GEMMA_TINY["vocab"], size=13)
    a, b = zq.Gemma3(host), zq.Gemma3(host)
    assert a.decode_mode == zq.DECODE_PERSISTENT
    b.set_decode_mode(zq.DECODE_LAUNCH_SEQUENCE)
    assert b.decode_mode == zq.DECODE_LAUNCH_SEQUENCE
    la, lb = a.prefill(prompt), b.prefill(prompt)
    assert torch.equal(la, lb)
    tok = int(la.argmax())
    for step in range(30):
        la, lb = a.decode_next(tok), b.decode_next(tok)
        assert torch.equal(la, lb), step
        tok = int(la.argmax())
    ta, tb = a.decode_greedy(tok, 25), b.decode_greedy(tok, 25)
    assert list(ta) == list(tb)
    assert a.seq_len == b.seq_len == 13 + 30 + 25
    # a single-token prefill and a cache-only step go through the kernel too
    a.reset_cache(), b.reset_cache()
    assert torch.equal(a.prefill([5]), b.prefill([5]))
    assert torch.equal(a.decode_next(7), b.decode_next(7))
    from zignn_b200 import _lib
    assert _lib.device_error(clear=False) == 0


def test_persistent_decode_kernel_full_size_greedy_against_launch_sequence(zq):
    """Gemma-3-1B shape, Q8_0, 600-token context (beyond the window): 48 greedy tokens from the on-device loop
    of the persistent kernel equal those of the launch sequence, and so do the logits of the step after."""
    host = hostmodel.Gemma3Host.synthetic(hostmodel.GEMMA3_1B, qtype=ggml.Q8_0, seed=42, std=0.02, device="cuda")
    prompt = np.random.default_rng(47).integers(0, 262144, size=600)
    a, b = zq.Gemma3(host), zq.Gemma3(host)
    b.set_decode_mode(zq.DECODE_LAUNCH_SEQUENCE)
    la, lb = a.prefill(prompt), b.prefill(prompt)
    assert torch.equal(la, lb)
    tok = int(la.argmax())
    ta, tb = a.decode_greedy(tok, 48), b.decode_greedy(tok, 48)
    assert list(ta) == list(tb)
    assert torch.equal(a.decode_next(int(ta[-1])), b.decode_next(int(tb[-1])))


def test_engines_from_gguf_files_match_engines_from_memory(zq, oracle, tmp_path):
    """Write the synthetic models as GGUF files under zig-nn's tensor names, map them back, and run the
    engines straight from the mapped bytes: logits are the bits of the in-memory model."""
    from zignn_b200 import gguf
    g_host = hostmodel.Gpt2Host.synthetic(GPT2_TINY, seed=42, std=0.08).randomize_small_params()
    g_path = str(tmp_path / "gpt2.gguf")
    g_host.to_gguf(g_path)
    prompt = np.random.default_rng(44).integers(0, GPT2_TINY["vocab"], size=20)
    a = zq.Gpt2(g_host).prefill(prompt).cpu().numpy()
    b = zq.Gpt2(hostmodel.Gpt2Host.from_gguf(g_path)).prefill(prompt).cpu().numpy()
    assert np.array_equal(a, b)

    m_host = hostmodel.Gemma3Host.synthetic(GEMMA_TINY, qtype=ggml.Q4_0, embd_qtype=ggml.Q8_0, down_qtype=ggml.Q4_1,
                                            seed=42, std=0.08).randomize_small_params()
    m_path = str(tmp_path / "gemma3.gguf")
    m_host.to_gguf(m_path)
    from_file = hostmodel.Gemma3Host.from_gguf(m_path)
    prompt = np.random.default_rng(45).integers(0, GEMMA_TINY["vocab"], size=24)
    eng = zq.Gemma3(from_file)
    ref = oracle.Gemma3(m_host, 4)
    lg, lc = eng.prefill(prompt).cpu().numpy(), ref.prefill(prompt)
    assert np.array_equal(lg, lc)
    for _ in range(8):
        t = int(np.argmax(lc))
        lg, lc = eng.decode_next(t).cpu().numpy(), ref.decode_next(t)
        assert np.array_equal(lg, lc)

    # a quantised tensor asked for as f32 is decoded by the CUDA decoder: the oracle's bits
    f = gguf.parse(m_path)
    r = f.get_tensor_raw_bytes("blk.0.ffn_down.weight")
    want = oracle.dequantize(r.type_, np.asarray(r.data), r.n_elem)
    assert np.array_equal(f.load_tensor_f32("blk.0.ffn_down.weight"), want)


@pytest.mark.parametrize("qtype", [ggml.Q4_0, ggml.Q4_1, ggml.Q8_0])
def test_gpt2_persistent_decode_kernel_against_the_launch_sequence(zq, qtype):
    """GPT-2 decode as one cooperative kernel per token against the captured launch sequence. This path's bar is
    a tolerance (f32 activations, no quantiser in the loop): logits agree to 1e-5 relative L2 step by step, the
    greedy tokens of the on-device loop are the same, and a run repeats itself bit for bit."""
    host = hostmodel.Gpt2Host.synthetic(GPT2_TINY, qtype=qtype, seed=5, std=0.08).randomize_small_params()
    prompt = np.random.default_rng(3).integers(0, GPT2_TINY["vocab"], size=13)
    a, b = zq.Gpt2(host), zq.Gpt2(host)
    assert a.decode_mode == zq.DECODE_PERSISTENT
    b.set_decode_mode(zq.DECODE_LAUNCH_SEQUENCE)
    assert b.decode_mode == zq.DECODE_LAUNCH_SEQUENCE
    la, lb = a.prefill(prompt), b.prefill(prompt)
    assert torch.equal(la, lb)  # prefill chunks take the batched path in both
    tok = int(la.argmax())
    first = tok
    for step in range(30):
        la, lb = a.decode_next(tok), b.decode_next(tok)
        assert rel_l2(la.cpu().numpy(), lb.cpu().numpy()) <= 1e-5, step
        assert int(la.argmax()) == int(lb.argmax()), step
        tok = int(lb.argmax())
    ta, tb = a.decode_greedy(tok, 25), b.decode_greedy(tok, 25)
    assert list(ta) == list(tb)
    assert a.seq_len == b.seq_len == 13 + 30 + 25
    # the same run again gives the same bits
    c = zq.Gpt2(host)
    c.prefill(prompt)
    tok = first
    for step in range(30):
        lc = c.decode_next(tok)
        tok = int(lc.argmax())
    assert torch.equal(lc, la)
    # a single-token prefill and a cache-only step go through the kernel too
    a.reset_cache(), b.reset_cache()
    assert rel_l2(a.prefill([5]).cpu().numpy(), b.prefill([5]).cpu().numpy()) <= 1e-5
    assert rel_l2(a.decode_next(7).cpu().numpy(), b.decode_next(7).cpu().numpy()) <= 1e-5
    from zignn_b200 import _lib
    assert _lib.device_error(clear=False) == 0


def test_gpt2_persistent_decode_kernel_full_size_greedy(zq):
    """GPT-2 small, Q4_0: 128 greedy tokens from the on-device loop of the persistent kernel equal those of the
    launch sequence (the workload of the decode benchmark)."""
    host = hostmodel.Gpt2Host.synthetic(hostmodel.GPT2_SMALL, qtype=ggml.Q4_0, seed=42, std=0.02, device="cuda")
    prompt = np.random.default_rng(44).integers(0, 50257, size=32)
    a, b = zq.Gpt2(host), zq.Gpt2(host)
    b.set_decode_mode(zq.DECODE_LAUNCH_SEQUENCE)
    la, lb = a.prefill(prompt), b.prefill(prompt)
    tok = int(la.argmax())
    ta, tb = a.decode_greedy(tok, 128), b.decode_greedy(tok, 128)
    assert list(ta) == list(tb)
    la, lb = a.decode_next(int(ta[-1])), b.decode_next(int(tb[-1]))
    assert rel_l2(la.cpu().numpy(), lb.cpu().numpy()) <= 1e-5
