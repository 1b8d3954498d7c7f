"""Decoder stack (config-4 structure at toy size) against a CPU restatement built from the oracle's pieces."""
import numpy as np
import pytest
import torch

from ojasx_b200 import inference_engine as ie

pytestmark = pytest.mark.gpu

CFG = ie.StackConfig(layers=2, hidden=128, q_heads=4, kv_heads=2, head_dim=32, experts=8, top_k=2, inter=64, vocab=300,
                     max_seq_len=32, distinct_layers=2, outlier_frac=0.01)


def _rms(x, w, eps):
    x = x.astype(np.float32)
    return (x * (np.float32(1.0) / np.sqrt((x * x).mean(dtype=np.float32) + np.float32(eps))) * w).astype(np.float32)


def _rope(x, pos, theta):
    hd = x.shape[-1]
    inv = (1.0 / (theta ** (np.arange(0, hd, 2, dtype=np.float32) / hd))).astype(np.float32)
    ang = (np.float32(pos) * inv).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    return np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).astype(np.float32)


class CpuStack:
    """One sequence, fp32, every VQ piece evaluated by the CPU oracle."""

    def __init__(self, O, W, cfg):
        self.O, self.W, self.cfg, self.pos = O, W, cfg, 0
        self.kc = [[np.zeros((0, cfg.head_dim // cfg.block_dim), np.uint8) for _ in range(cfg.kv_heads)] for _ in range(cfg.layers)]
        self.vc = [[np.zeros((0, cfg.head_dim // cfg.block_dim), np.uint8) for _ in range(cfg.kv_heads)] for _ in range(cfg.layers)]

    def lin(self, w, x):
        return self.O.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=self.cfg.block_dim)

    def step(self, tok):
        O, cfg = self.O, self.cfg
        R = cfg.q_heads // cfg.kv_heads
        h = self.W.embed[tok].copy()
        for li in range(cfg.layers):
            w = self.W.layers[li % len(self.W.layers)]
            a = _rms(h, w.norm1, cfg.rms_eps)
            q = _rope(self.lin(w.q, a).reshape(cfg.q_heads, cfg.head_dim), self.pos, cfg.rope_theta)
            k = _rope(self.lin(w.k, a).reshape(cfg.kv_heads, cfg.head_dim), self.pos, cfg.rope_theta)
            v = self.lin(w.v, a).reshape(cfg.kv_heads, cfg.head_dim)
            att = np.zeros((cfg.q_heads, cfg.head_dim), np.float32)
            for kh in range(cfg.kv_heads):
                self.kc[li][kh] = np.concatenate([self.kc[li][kh], O.kvq_encode(k[kh], w.k_codebook[kh], block_dim=cfg.block_dim)[None]])
                self.vc[li][kh] = np.concatenate([self.vc[li][kh], O.kvq_encode(v[kh], w.v_codebook[kh], block_dim=cfg.block_dim)[None]])
                att[kh * R:(kh + 1) * R] = O.kvq_decode(q[kh * R:(kh + 1) * R], self.kc[li][kh], self.vc[li][kh],
                                                        w.k_codebook[kh], w.v_codebook[kh], block_dim=cfg.block_dim)
            h = (h + self.lin(w.o, att.reshape(-1))).astype(np.float32)
            m = _rms(h, w.norm2, cfg.rms_eps)
            idx, wt = O.router_topk(m, w.moe.router, cfg.top_k)
            mo = w.moe
            h = (h + O.moe_forward(mo.codebook, mo.down_codebook, mo.gate_up_codes, mo.gate_up_scales, mo.down_codes,
                                   mo.down_scales, m, idx[0], wt[0], block_dim=cfg.block_dim, gu_csr=mo.gate_up_csr,
                                   dn_csr=mo.down_csr)).astype(np.float32)
        self.pos += 1
        return self.lin(self.W.lm_head, _rms(h, self.W.final_norm, cfg.rms_eps))


def test_decoder_stack_logits_and_greedy_tokens(cuda, oracle):
    W = ie.make_stack_weights(11, CFG)
    stack = ie.VQDecoderStack(W, CFG, batch=2)
    prompt = np.array([[5, 17, 250, 3], [9, 9, 120, 44]], np.int64)
    cpu = [CpuStack(oracle, W, CFG) for _ in range(2)]
    for s in range(prompt.shape[1]):
        got = stack.decode_step(torch.from_numpy(prompt[:, s])).cpu().numpy()
        for b in range(2):
            want = cpu[b].step(int(prompt[b, s]))
            assert np.allclose(got[b], want, rtol=2e-3, atol=2e-4), (s, b, np.abs(got[b] - want).max())
    # greedy continuation through the engine's public call equals the CPU stack's arg-max chain
    eng = ie.UniversalInferenceEngine(stack)
    ids = eng.generate(torch.from_numpy(prompt).to(cuda), max_new_tokens=3).cpu().numpy()
    for b in range(2):
        ref = CpuStack(oracle, W, CFG)
        logits = None
        for t in prompt[b]:
            logits = ref.step(int(t))
        for j in range(3):
            nxt = int(np.argmax(logits))
            assert ids[b, j] == nxt, (b, j)
            logits = ref.step(nxt)
    with pytest.raises(ValueError):
        eng.generate(torch.from_numpy(prompt).to(cuda), max_new_tokens=40)


def test_decoder_stack_graph_replay_equals_eager(cuda):
    """One captured decode step replayed per token gives the same logits as the eager launch sequence."""
    W = ie.make_stack_weights(12, CFG)
    eager = ie.VQDecoderStack(W, CFG, batch=2)
    graph = ie.VQDecoderStack(W, CFG, batch=2, use_graph=True)
    toks = np.random.default_rng(0).integers(0, CFG.vocab, size=(2, 9))
    for s in range(toks.shape[1]):
        ids = torch.from_numpy(toks[:, s])
        a = eager.decode_step(ids)
        b = graph.decode_step(ids).clone()
        assert torch.equal(a, b), s
    assert graph.layers[0].cache.sync_len() == 9


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batched_prefill_equals_token_by_token(cuda, dtype):
    """The prompt as one batch through the linears and the MoE (attention position by position) leaves the same
    caches and logits as feeding it token by token; a captured decode step can start on the prefilled caches."""
    W = ie.make_stack_weights(13, CFG)
    toks = torch.from_numpy(np.random.default_rng(1).integers(0, CFG.vocab, size=(2, 11))).to(cuda)
    one = ie.VQDecoderStack(W, CFG, batch=2, dtype=dtype)
    ref = one.prefill(toks, batched=False)
    for graph in (False, True):
        st = ie.VQDecoderStack(W, CFG, batch=2, dtype=dtype, use_graph=graph)
        got = st.prefill(toks, max_rows=8)            # three chunks of four, four and three positions
        if dtype == torch.float32:
            assert torch.equal(got, ref)
        else:                                           # bf16 batches may take another kernel than single tokens
            assert torch.allclose(got, ref, rtol=5e-2, atol=5e-2)
        assert st.layers[1].cache.sync_len() == 11 and st.position == 11
        nxt = torch.argmax(ref, dim=-1)
        a, b = st.decode_step(nxt).clone(), one.decode_step(nxt)
        if dtype == torch.float32:
            assert torch.equal(a, b), graph
        assert st.layers[0].cache.sync_len() == 12
        one.reset()
        one.prefill(toks, batched=False)
