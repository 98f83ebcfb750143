"""Decoder harness on one GPU: the graph-captured decode step reproduces the eager one, and the
quantised model agrees with the same model evaluated on dense dequantised weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from autogptq.tvm_b200 import decoder, ops
    DEV = torch.device("cuda:0")


def _small(arch, bits, desc_act):
    return decoder.DecoderConfig(arch=arch, layers=2, hidden=256, heads=4, inter=512, vocab=1000, bits=bits,
                                 group_size=128, desc_act=desc_act, max_seq=64)


@pytest.mark.parametrize("arch,bits,desc_act", [("llama", 4, False), ("opt", 3, True)])
def test_graph_decode_equals_eager_decode(arch, bits, desc_act):
    cfg = _small(arch, bits, desc_act)
    prompt = torch.randint(0, cfg.vocab, (1, 12), generator=torch.Generator().manual_seed(1)).to(DEV)
    a = decoder.GPTQDecoder(cfg, batch=1, device=DEV)
    a.prefill(prompt)
    eager = a.decode(6).cpu()
    b = decoder.GPTQDecoder(cfg, batch=1, device=DEV)
    b.prefill(prompt)
    b.capture()
    graphed = b.decode(6).cpu()
    assert torch.equal(eager, graphed)
    assert int(b.pos) == 12 + 6


@pytest.mark.parametrize("arch,bits,desc_act", [("llama", 4, False), ("opt", 3, True)])
def test_tuning_in_place_keeps_the_state_and_the_result(arch, bits, desc_act):
    """GPTQDecoder.tune(): every kind of linear gets one of the candidate work splits, position and tokens are as
    before, and the logits of the next step stay within the output contract of the untuned decoder's (a different
    split of K changes the order of the fp32 sums only)."""
    cfg = _small(arch, bits, desc_act)
    prompt = torch.randint(0, cfg.vocab, (1, 12), generator=torch.Generator().manual_seed(1)).to(DEV)
    ref = decoder.GPTQDecoder(cfg, batch=1, device=DEV)
    ref.prefill(prompt)
    ref.decode(1)
    m = decoder.GPTQDecoder(cfg, batch=1, device=DEV)
    m.prefill(prompt)
    pos, tok = int(m.pos), m.tokens.clone()
    chosen = m.tune(steps=4)
    assert set(chosen) == {"qkv", "o", "up", "down"} and all(c in m.TUNINGS for c in chosen.values())
    assert int(m.pos) == pos and torch.equal(m.tokens, tok) and m._pos_host == pos
    for L in m.layers:
        assert L.qkv.gemv_tuning == chosen["qkv"] and L.down.gemv_tuning == chosen["down"]
    m.decode(1)
    assert torch.allclose(m.last_logits.float(), ref.last_logits.float(), rtol=0, atol=2e-2)
    ops.check_status(DEV)


class _Dense(torch.nn.Module):
    """Stand-in for a QuantLinear that multiplies by the dequantised fp16 weights with torch."""

    def __init__(self, q):
        super().__init__()
        g = q._g_idx_run if q._g_idx_run is not None else \
            (torch.arange(q.infeatures, device=q.qweight.device) // q.groupsize).to(torch.int32)
        _, W = ops.dequantize(q._qweight_run, q.qzeros, q.scales, g, q.bits, q.groupsize, want_q=False)
        self.W, self.bias, self.perm = W.float(), q.bias, q._x_perm

    def forward(self, x):
        xf = x.float()
        if self.perm is not None:
            xf = xf[:, self.perm.long()]
        y = xf @ self.W
        if self.bias is not None:
            y = y + self.bias.float()
        return y.half()


@pytest.mark.parametrize("arch,bits,desc_act", [("llama", 4, False), ("opt", 3, True)])
def test_quantised_model_matches_dense_model(arch, bits, desc_act):
    cfg = _small(arch, bits, desc_act)
    prompt = torch.randint(0, cfg.vocab, (2, 20), generator=torch.Generator().manual_seed(2)).to(DEV)
    q = decoder.GPTQDecoder(cfg, batch=2, device=DEV)
    d = decoder.GPTQDecoder(cfg, batch=2, device=DEV)   # same seeds => same weights
    for L in d.layers:
        L.qkv, L.o, L.up, L.down = _Dense(L.qkv), _Dense(L.o), _Dense(L.up), _Dense(L.down)
    pos = torch.arange(20, device=DEV)
    xq, xd = q._embed(prompt, pos), d._embed(prompt, pos)
    for Lq, Ld in zip(q.layers, d.layers):
        xq = q._layer(Lq, xq, pos, 20, decode=False)
        xd = d._layer(Ld, xd, pos, 20, decode=False)
    err = (xq.float() - xd.float()).abs().max().item()
    scale = xd.float().abs().max().item()
    assert err <= 2e-2 * max(scale, 1.0), (err, scale)


@pytest.mark.parametrize("arch,bits,desc_act", [("llama", 4, False), ("opt", 3, True)])
def test_fused_decode_step_matches_the_framework_ops(arch, bits, desc_act):
    """The fused helper kernels (norm, rotary + cache write, single-query attention, activation) against the
    same step written with torch ops: same residual stream, within fp16 round-off of the attention."""
    cfg = _small(arch, bits, desc_act)
    prompt = torch.randint(0, cfg.vocab, (2, 10), generator=torch.Generator().manual_seed(4)).to(DEV)
    a = decoder.GPTQDecoder(cfg, batch=2, device=DEV, fused=True)
    b = decoder.GPTQDecoder(cfg, batch=2, device=DEV, fused=False)
    a.prefill(prompt)
    b.prefill(prompt)
    assert torch.equal(a.tokens, b.tokens)
    for _ in range(4):
        a._decode_step()
        b._decode_step()
    for La, Lb in zip(a.layers, b.layers):   # what the steps wrote into the caches
        ka, kb = La.k_cache[:, :, :14].float(), Lb.k_cache[:, :, :14].float()
        va, vb = La.v_cache[:, :, :14].float(), Lb.v_cache[:, :, :14].float()
        assert (ka - kb).abs().max() <= 2e-2 * max(kb.abs().max().item(), 1.0)
        assert (va - vb).abs().max() <= 2e-2 * max(vb.abs().max().item(), 1.0)


@pytest.mark.parametrize("M,K,N", [(1, 4096, 32000), (3, 4096, 4001), (8, 1024, 517), (1, 9216, 50272 // 8)])
def test_dense_gemv_matches_fp32_product(M, K, N):
    """Vocabulary projection: fp16 in, fp32 sums of 8-product fp16 partial sums, fp16 out, against the fp64 product."""
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g).half()
    w = (0.02 * torch.randn(N, K, generator=g)).half()
    y = ops.dense_gemv(x.to(DEV), w.to(DEV))
    ref = x.double() @ w.double().t()
    err = (y.cpu().double() - ref).abs()
    # one fp16 rounding of the result plus the half-precision partial sums: 2^-10 relative to sum |x w|
    bound = 2.0 ** -10 * (x.double().abs() @ w.double().abs().t()) + 1e-4
    assert bool((err <= bound).all()), float((err / bound).max())
    assert torch.equal(y, ops.dense_gemv(x.to(DEV), w.to(DEV)))
    with pytest.raises(ValueError):
        ops.dense_gemv(torch.zeros(9, K, dtype=torch.float16, device=DEV), w.to(DEV))


@pytest.mark.parametrize("arch,bits,desc_act,batch", [("llama", 4, False, 1), ("opt", 3, True, 1), ("llama", 4, False, 4)])
def test_folded_activation_gives_the_same_tokens(arch, bits, desc_act, batch):
    """The second FFN linear applying SiLU(gate) * up / ReLU as it reads its input (one launch fewer per layer) is
    bit-identical to the separate element-wise kernel: same logits, same tokens."""
    cfg = _small(arch, bits, desc_act)
    prompt = torch.randint(0, cfg.vocab, (batch, 9), generator=torch.Generator().manual_seed(3)).to(DEV)
    outs = []
    for fold in (True, False):
        m = decoder.GPTQDecoder(cfg, batch=batch, device=DEV, fold_activation=fold)
        m.prefill(prompt)
        m.capture()
        toks = m.decode(5).cpu()
        outs.append((toks, m.last_logits.cpu()))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])
    m = decoder.GPTQDecoder(cfg, batch=batch, device=DEV, fold_activation=True)
    folds = [L.down.can_fold(batch, 1 if arch == "llama" else 2) for L in m.layers]
    assert all(folds), "the miniature's FFN layers are expected to take the folded activation"


@pytest.mark.parametrize("rows,ld,valid", [(1, 32000, 32000), (3, 4000, 3997), (16, 1000, 1000), (2, 8, 5)])
def test_greedy_pick_matches_argmax(rows, ld, valid):
    """b200gptq_pick_local on one rank: the framework's argmax over the valid columns (first maximum on ties, which
    fp16 logits do produce), clamped, and the position advanced by one.  And the two-launch form for several ranks,
    emulated on one GPU: each "rank" fills its slots of its own vector, their sum goes through b200gptq_pick_final."""
    g = torch.Generator().manual_seed(rows + ld)
    logits = (4 * torch.randn(rows, ld, generator=g)).half().to(DEV)
    logits[0, valid // 2] = logits[0, : valid].max()          # a tie: the lower column wins
    logits[:, valid:] = 1e4                                   # padding columns never win
    tokens = torch.zeros(rows, dtype=torch.long, device=DEV)
    pos = torch.tensor([41], dtype=torch.long, device=DEV)
    ops.pick_local(logits, valid, 0, 1, 0, None, tokens, valid - 1, pos)
    want = logits[:, :valid].float().argmax(dim=-1)
    assert torch.equal(tokens, want) and int(pos) == 42
    # four emulated ranks, each holding a quarter of the columns (the last one with padding)
    world, per = 4, ld // 4 // 8 * 8
    if per >= 8:
        total = torch.zeros(rows, 4 * world, dtype=torch.float32, device=DEV)
        for r in range(world):
            part = logits[:, r * per:(r + 1) * per].contiguous()
            v = max(1, min(per, valid - r * per))
            slots = torch.full((rows, 4 * world), 7.0, dtype=torch.float16, device=DEV)
            ops.pick_local(part, v, r * per, world, r, slots, None, valid - 1)
            total += slots.float()
        out = torch.zeros(rows, dtype=torch.long, device=DEV)
        ops.pick_final(total.half(), world, out, valid - 1, pos)
        cols = min(valid, world * per)
        assert torch.equal(out, logits[:, :cols].float().argmax(dim=-1)) and int(pos) == 43


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("B,heads,pos", [(1, 8, 200), (2, 30, 200), (4, 30, 97), (8, 30, 255), (16, 24, 130), (3, 5, 0)])
def test_single_query_attention_matches_fp32_softmax(hd, B, heads, pos):
    """b200gptq_attn_decode against softmax(q k^T / sqrt(hd)) v in fp32, for every way the launcher divides the work:
    from a cluster of four 16-warp CTAs per (sequence, head) for one sequence down to one 4-warp CTA for a batch."""
    max_seq = 256
    g = torch.Generator().manual_seed(hd + pos + B)
    q = torch.randn(B, heads * hd, generator=g).half().to(DEV)
    kc = torch.randn(B, heads, max_seq, hd, generator=g).half().to(DEV)
    vc = torch.randn(B, heads, max_seq, hd, generator=g).half().to(DEV)
    p = torch.tensor([pos], dtype=torch.long, device=DEV)
    got = ops.attn_decode(q, kc, vc, p, torch.empty_like(q), heads, hd)
    qf = q.float().reshape(B, heads, 1, hd)
    sc = (qf @ kc[:, :, :pos + 1].float().transpose(2, 3)) / hd ** 0.5
    want = (torch.softmax(sc, dim=-1) @ vc[:, :, :pos + 1].float()).reshape(B, heads * hd)
    assert torch.allclose(got.float(), want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("hd,rope,B,heads,pos", [(128, True, 1, 4, 37), (64, False, 3, 6, 0), (128, True, 2, 3, 255), (64, True, 1, 2, 100),
                                                 (128, True, 16, 24, 130), (64, True, 8, 30, 70), (128, False, 4, 30, 33), (128, True, 2, 30, 200)])
def test_attention_step_equals_its_two_kernels(hd, rope, B, heads, pos):
    """b200gptq_attn_step (rotary + cache write + attention in one launch) against b200gptq_rope_cache followed by
    b200gptq_attn_decode: the same caches bit for bit, the same attention output up to the order in which the new
    position enters the online softmax."""
    max_seq = 256
    g = torch.Generator().manual_seed(hd + pos)
    qkv = torch.randn(B, 3 * heads * hd, generator=g).half().to(DEV)
    kc = torch.randn(B, heads, max_seq, hd, generator=g).half().to(DEV)
    vc = torch.randn(B, heads, max_seq, hd, generator=g).half().to(DEV)
    ang = torch.arange(max_seq).float()[:, None] * (1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd)))[None, :]
    cos, sin = ang.cos().half().to(DEV), ang.sin().half().to(DEV)
    p = torch.tensor([pos], dtype=torch.long, device=DEV)
    k1, v1 = kc.clone(), vc.clone()
    q = torch.empty(B, heads * hd, dtype=torch.float16, device=DEV)
    ops.rope_cache(qkv, cos, sin, p, q, k1, v1, heads, hd, rope)
    want = ops.attn_decode(q, k1, v1, p, torch.empty_like(q), heads, hd)
    k2, v2 = kc.clone(), vc.clone()
    got = ops.attn_step(qkv, cos, sin, p, k2, v2, torch.empty_like(q), heads, hd, rope)
    assert torch.allclose(got.float(), want.float(), rtol=2e-3, atol=2e-3)
    assert torch.equal(k2, k1) and torch.equal(v2, v1)
    # a position outside the caches is refused without touching them
    bad = torch.tensor([max_seq], dtype=torch.long, device=DEV)
    k3 = kc.clone()
    ops.attn_step(qkv, cos, sin, bad, k3, vc.clone(), torch.empty_like(q), heads, hd, rope)
    assert torch.equal(k3, kc)
