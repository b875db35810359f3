"""Rotation kernel, loader, decoder and graph wrapper on the GPU against the CPU oracle.

Bars: low-rank factors read from a checkpoint bit-identical to the oracle's; rotated activations
within 1e-6 (fp32) / one fp16 rounding; logits of a two-layer decoder within rel-L2 5e-3 of the
oracle's full causal forward (each quantized layer is held to 1e-3 on its own; attention runs
through the library's fused kernel with fp32 accumulation where the oracle rounds the probabilities
to fp16)."""

import pytest
import torch

from oracle import glorcq_oracle as O
from tests import cases

pytestmark = pytest.mark.gpu
REL_LOGITS = 5e-3

CFG = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=512,
           num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=256,
           norm_topk_prob=False, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=64)
MIXTRAL = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=300,
               num_local_experts=4, num_experts_per_tok=2, intermediate_size=384, rms_norm_eps=1e-5,
               rope_theta=1e6, max_position_embeddings=64)
QWEN3 = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
             vocab_size=300, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128, norm_topk_prob=True,
             rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=64)


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from glorcq_b200 import _build
    _build.build()
    return torch.device("cuda:0")


@pytest.mark.parametrize("d", [2048, 1408, 768, 64, 48])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_rht_forward(dev, d, dtype):
    from glorcq_b200.hadamard_rotation import generate_rht_signs, rht_backward, rht_forward, rht_forward_half
    x = cases.make_x(900 + d, 5, d, dtype)
    signs = generate_rht_signs(d, seed=d, device=dev)
    ref = O.rht_forward(x.float(), O.generate_rht_signs(d, d))
    y = rht_forward(x.to(dev), signs)
    assert y.dtype == dtype and y.shape == x.shape
    if dtype == torch.float32:
        assert torch.allclose(y.cpu(), ref, atol=2e-6 * d ** 0.5)
        if d & (d - 1) == 0:
            assert torch.allclose(rht_backward(y, signs).cpu(), x, atol=1e-5)
    else:
        assert cases.rel_l2(y.cpu(), ref) <= 5e-4
    yh = rht_forward_half(x.to(dev), signs)
    assert yh.dtype == torch.float16 and cases.rel_l2(yh.cpu(), ref) <= 5e-4
    assert rht_forward(x[:0].to(dev), signs).shape == (0, d)


@pytest.mark.parametrize("N", [1, 6, 70])
def test_codebook_block_with_hadamard_rotation(dev, N):
    blk = cases.make_moe(36, 256, 128, 6, 2, I_shared=256, rank=16, experts_per_cluster=2, fmt="turbo")
    for ex in blk["experts"] + [blk["shared_expert"]]:
        for p in ex.values():
            p["Pi"] = None
            p["rht_seed"] = 42
    mb = cases.to_b200_moe(blk, dev)
    x = cases.make_x(1036 + N, N, 256).reshape(1, N, 256)
    y, _ = mb(x.to(dev))
    ref, _ = O.moe_forward(cases.to_oracle_moe(blk), x)
    assert cases.rel_l2(y.cpu(), ref) <= 2e-3


def _models(cfg, dev, seed, **kw):
    from glorcq_b200 import model_builder as MB
    from glorcq_b200 import synthetic
    from glorcq_b200.decoder import GLoRCQDecoder
    md, cr, dense = synthetic.make_checkpoint(cfg, seed=seed, rank=16, attn_rank=32, n_clusters=3, **kw)
    layers, u_cache = MB.build_layers(md["model_config"], md["layers"], cr, device=dev)
    return GLoRCQDecoder(cfg, layers, dense=dense, device=dev), layers, O.checkpoint_layers(md, cr), dense


@pytest.mark.parametrize("fmt", ["int4", "fp16", "int8"])
def test_build_layers_matches_oracle(dev, fmt):
    model, layers, olayers, _ = _models(CFG, dev, 21, u_format=fmt, sv_format=fmt)
    for name in ("self_attn.q_proj", "mlp.experts.3.down_proj", "mlp.experts.0.gate_proj", "mlp.shared_expert.up_proj"):
        ql, oq = layers[1][name], olayers[1][name]
        if oq.U is None:
            assert ql.U is None and ql.SV is None
        else:
            assert torch.equal(ql.U.cpu(), oq.U) and torch.equal(ql.SV.cpu(), oq.SV)
            assert tuple(ql.cluster_id) == tuple(oq.cluster_id)
    # layers of one cluster share one U tensor (and so one tiled copy)
    by_cluster = {}
    for mods in layers.values():
        for ql in mods.values():
            if ql.U is not None:
                by_cluster.setdefault(ql.cluster_id, set()).add(ql.U.data_ptr())
    assert all(len(v) == 1 for v in by_cluster.values())
    x = cases.make_x(5, 3, 256)
    ql, oq = layers[0]["self_attn.o_proj"], olayers[0]["self_attn.o_proj"]
    assert cases.rel_l2(ql(x.to(dev)).cpu(), O.linear_forward(oq, x)) <= 1e-3


def test_build_layers_dense_and_unknown_records(dev):
    """A ``weight_quant`` record (pre-dequantised weights) loads as a dense layer with its low-rank factors, an
    unknown record is skipped, as the reference's loader does (inference/model_builder.py:380-415)."""
    from glorcq_b200 import model_builder as MB
    from glorcq_b200 import synthetic
    md, cr, _ = synthetic.make_checkpoint(CFG, seed=23, rank=16, attn_rank=32, n_clusters=3, u_format="fp16", sv_format="fp16")
    rec = md["layers"][0]["self_attn.o_proj"]
    W = O.gptq_tile_fp16(rec["qweight_int"], rec["scales"], rec["zeros"], rec["groupsize"])
    md["layers"][0]["self_attn.o_proj"] = {"weight_quant": W, "quant_method": "rtn"}
    md["layers"][0]["mlp.experts.0.up_proj"] = {"something_else": torch.zeros(1)}
    layers, _ = MB.build_layers(md["model_config"], md["layers"], cr, device=dev)
    assert "mlp.experts.0.up_proj" not in layers[0]
    ql = layers[0]["self_attn.o_proj"]
    assert ql.quant_type == "rtn" and ql.SV is not None
    x = cases.make_x(6, 3, 256)
    oq = O.checkpoint_layers({"model_config": md["model_config"], "layers": {0: {"self_attn.o_proj": rec}}}, cr)[0]["self_attn.o_proj"]
    assert cases.rel_l2(ql(x.to(dev)).cpu(), O.linear_forward(oq, x)) <= 1e-3


@pytest.mark.parametrize("cache_len", [32, 320])     # 320: the decode attention splits the positions over CTAs
@pytest.mark.parametrize("cfg", [CFG, MIXTRAL, QWEN3], ids=["qwen2moe", "mixtral", "qwen3moe"])
def test_decoder_logits_prefill_and_decode(dev, cfg, cache_len):
    from glorcq_b200.decoder import StaticKVCache
    model, _, olayers, dense = _models(cfg, dev, 31)
    if cfg is QWEN3:   # per-head q/k norms
        g = torch.Generator().manual_seed(7)
        for l in range(2):
            dense[f"model.layers.{l}.self_attn.q_norm.weight"] = (1 + 0.1 * torch.randn(32, generator=g)).half()
            dense[f"model.layers.{l}.self_attn.k_norm.weight"] = (1 + 0.1 * torch.randn(32, generator=g)).half()
        from glorcq_b200 import model_builder as MB
        from glorcq_b200 import synthetic
        from glorcq_b200.decoder import GLoRCQDecoder
        md, cr, _ = synthetic.make_checkpoint(cfg, seed=31, rank=16, attn_rank=32, n_clusters=3)
        layers, _ = MB.build_layers(md["model_config"], md["layers"], cr, device=dev)
        model = GLoRCQDecoder(cfg, layers, dense=dense, device=dev)
    T = 12 if cache_len == 32 else 45
    ids = torch.randint(0, cfg["vocab_size"], (1, T + 1), generator=torch.Generator().manual_seed(3))
    ref = O.decoder_forward(cfg, olayers, dense, ids)
    cache = StaticKVCache(model.config, 1, cache_len, dev)
    with torch.no_grad():
        lg = model(input_ids=ids[:, :T].to(dev), cache_position=torch.arange(T, device=dev), past_key_values=cache)[0]
        assert cases.rel_l2(lg.cpu(), ref[:, :T]) <= REL_LOGITS
        step = model(input_ids=ids[:, T:].to(dev), cache_position=torch.tensor([T], device=dev), past_key_values=cache)[0]
    assert step.shape == (1, 1, cfg["vocab_size"])
    assert cases.rel_l2(step.cpu(), ref[:, T:]) <= REL_LOGITS


@pytest.mark.parametrize("B,T,nh,nkv,hd,norms", [(1, 37, 4, 4, 128, False), (2, 19, 8, 2, 64, True), (1, 5, 2, 1, 32, True)])
def test_rope_prefill_matches_tensor_ops(dev, B, T, nh, nkv, hd, norms):
    """The prompt's norms + rotary embedding + cache write in one launch against the fp16 tensor operations it
    replaces (same roundings: bit-equal), with positions that are not 0..T-1 and grouped-query head counts."""
    import torch.nn.functional as F
    from glorcq_b200 import _lib, tiled
    from glorcq_b200.decoder import _rope_tables, _rotate_half
    g = torch.Generator().manual_seed(B * 1000 + T)
    max_len = 64
    q = torch.randn(B, T, nh, hd, generator=g).half().to(dev)
    k = torch.randn(B, T, nkv, hd, generator=g).half().to(dev)
    v = torch.randn(B, T, nkv, hd, generator=g).half().to(dev)
    qw = (torch.rand(hd, generator=g) + 0.5).half().to(dev) if norms else None
    kw = (torch.rand(hd, generator=g) + 0.5).half().to(dev) if norms else None
    pos = (torch.randperm(max_len, generator=g)[:T]).to(dev)
    cos, sin = _rope_tables(hd, max_len, 10000.0, dev)
    qr, kr = q, k
    if norms:
        qr, kr = F.rms_norm(q, (hd,), qw, 1e-6), F.rms_norm(k, (hd,), kw, 1e-6)
    cs, sn = cos[pos][None, :, None], sin[pos][None, :, None]
    qr = qr * cs + _rotate_half(qr) * sn
    kr = kr * cs + _rotate_half(kr) * sn
    kc = torch.zeros(B, nkv, max_len, hd, dtype=torch.float16, device=dev)
    vc = torch.zeros_like(kc)
    q2, k2 = q.clone(), k.clone()
    _lib.check(_lib.lib().glq_rope_prefill(q2.data_ptr(), k2.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                           pos.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, T, nh, nkv, hd, max_len,
                                           None if qw is None else qw.data_ptr(), None if kw is None else kw.data_ptr(),
                                           1e-6, tiled._stream_ptr(dev)), "rope_prefill")
    torch.cuda.synchronize()
    assert torch.equal(q2, qr) and torch.equal(k2, kr)
    assert torch.equal(kc[:, :, pos], kr.transpose(1, 2)) and torch.equal(vc[:, :, pos], v.transpose(1, 2))
    rest = torch.ones(max_len, dtype=torch.bool, device=dev)
    rest[pos] = False
    assert not kc[:, :, rest].any() and not vc[:, :, rest].any()


@pytest.mark.parametrize("B,T,nh,nkv,hd", [(1, 1, 2, 2, 128), (2, 200, 4, 2, 128), (1, 64, 2, 2, 64), (1, 513, 16, 16, 128),
                                          (3, 65, 8, 2, 64), (1, 1031, 4, 1, 128)])
def test_attn_prefill_matches_fp32_attention(dev, B, T, nh, nkv, hd):
    """The prompt's causal attention kernel (grouped-query head counts, lengths off the 64-row blocks) against
    softmax(q k^T / sqrt(hd)) v in fp32 on the same fp16 operands; fp16 probabilities and outputs in the kernel:
    rel-L2 <= 2e-3 and every element within 4e-3 of the row's largest magnitude."""
    from glorcq_b200 import _lib, tiled
    g = torch.Generator().manual_seed(T * 7 + nh)
    q = torch.randn(B, T, nh, hd, generator=g).half().to(dev)
    k = torch.randn(B, T, nkv, hd, generator=g).half().to(dev)
    v = torch.randn(B, T, nkv, hd, generator=g).half().to(dev)
    y = torch.full_like(q, float("nan"))
    _lib.check(_lib.lib().glq_attn_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), B, T, nh, nkv, hd,
                                           tiled._stream_ptr(dev)), "attn_prefill")
    torch.cuda.synchronize()
    qf = q.float().transpose(1, 2)                                              # (B, nh, T, hd)
    kf = k.float().transpose(1, 2).repeat_interleave(nh // nkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(nh // nkv, dim=1)
    s = qf @ kf.transpose(-1, -2) / hd ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=dev), 1), float("-inf"))
    ref = (torch.softmax(s, -1) @ vf).transpose(1, 2)                           # (B, T, nh, hd)
    assert torch.isfinite(y).all()
    assert cases.rel_l2(y.cpu(), ref.cpu()) <= 2e-3
    assert ((y.float() - ref).abs() <= 4e-3 * ref.abs().amax(-1, keepdim=True) + 1e-4).all()
    assert _lib.lib().glq_attn_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), B, T, nh, nkv, 96,
                                       tiled._stream_ptr(dev)) == -3       # GLQ_ERR_UNSUPPORTED


@pytest.mark.parametrize("B,V,H", [(1, 151936, 2048), (8, 151936, 2048), (3, 1000, 64), (5, 32000, 4096), (1, 17, 32)])
def test_lm_head_logits_and_argmax(dev, B, V, H):
    """glq_lm_head through the C ABI against the fp32 product of the same fp16 operands: logits within one
    fp16 rounding (rel-L2 <= 1e-3), arg-max = lowest index of the largest fp16-rounded logit, twice in a row
    (the arrival counter must be left zero)."""
    from glorcq_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(B + V + H)
    W = (torch.randn(V, H, generator=g) * 0.02).half().to(dev)
    x = torch.randn(B, H, generator=g).half().to(dev)
    ref = (x.float() @ W.float().t())
    ws = torch.empty(L.glq_lm_head_workspace_bytes(), dtype=torch.uint8, device=dev)
    ctr = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        logits = torch.full((B, V), float("nan"), dtype=torch.float16, device=dev)
        best = torch.full((B,), -1, dtype=torch.int64, device=dev)
        _lib.check(L.glq_lm_head(x.data_ptr(), H, W.data_ptr(), B, V, H, logits.data_ptr(), V, best.data_ptr(),
                                 ws.data_ptr(), ws.numel(), ctr.data_ptr(), st), "lm_head")
        torch.cuda.synchronize()
        assert int(ctr) == 0
        assert cases.rel_l2(logits.cpu(), ref.cpu()) <= 1e-3
        assert torch.equal(best, torch.argmax(logits, dim=-1))
    # arg-max only, and logits only
    best2 = torch.full((B,), -1, dtype=torch.int64, device=dev)
    _lib.check(L.glq_lm_head(x.data_ptr(), H, W.data_ptr(), B, V, H, None, 0, best2.data_ptr(), ws.data_ptr(), ws.numel(),
                             ctr.data_ptr(), st), "lm_head")
    assert torch.equal(best2, best)
    logits2 = torch.empty_like(logits)
    _lib.check(L.glq_lm_head(x.data_ptr(), H, W.data_ptr(), B, V, H, logits2.data_ptr(), V, None, None, 0, None, st), "lm_head")
    assert torch.equal(logits2, logits)
    assert L.glq_lm_head(x.data_ptr(), H, W.data_ptr(), 9, V, H, logits2.data_ptr(), V, None, None, 0, None, st) == -3


QWEN15_SHAPE = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=16,
                    vocab_size=151936, num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408,
                    shared_expert_intermediate_size=5632, norm_topk_prob=False, rms_norm_eps=1e-6,
                    rope_theta=1000000.0, max_position_embeddings=64)


@pytest.mark.timeout(1200)
def test_decoder_logits_at_qwen15_moe_dimensions(dev):
    """Two layers of the Qwen1.5-MoE-A2.7B shape at its own dimensions (hidden 2048, 16 heads of 128, 60
    experts top-4 x 1408 + shared expert 5632, vocabulary 151936; attention 4-bit, experts 2-bit, rank 64, 128
    cross-layer U clusters): logits of a 6-token prefill and of one decode step against the oracle's causal
    forward, rel-L2 <= 5e-3, and the same greedy token."""
    from glorcq_b200 import model_builder as MB
    from glorcq_b200 import synthetic
    from glorcq_b200.decoder import GLoRCQDecoder, StaticKVCache
    cfg = QWEN15_SHAPE
    md, cr, dense = synthetic.make_checkpoint(cfg, seed=51, rank=64, attn_rank=64, n_clusters=128, u_format="fp16",
                                              sv_format="fp16")
    layers, _ = MB.build_layers(md["model_config"], md["layers"], cr, device=dev)
    model = GLoRCQDecoder(cfg, layers, dense=dense, device=dev)
    T = 6
    ids = torch.randint(0, cfg["vocab_size"], (1, T + 1), generator=torch.Generator().manual_seed(13))
    cache = StaticKVCache(model.config, 1, 32, dev)
    with torch.no_grad():
        lg = model(input_ids=ids[:, :T].to(dev), cache_position=torch.arange(T, device=dev), past_key_values=cache)[0].cpu()
        step = model(input_ids=ids[:, T:].to(dev), cache_position=torch.tensor([T], device=dev), past_key_values=cache)[0].cpu()
    del model, layers
    torch.cuda.empty_cache()
    ref = O.decoder_forward(cfg, O.checkpoint_layers(md, cr), dense, ids)
    assert step.shape == (1, 1, cfg["vocab_size"])
    assert cases.rel_l2(lg, ref[:, :T]) <= REL_LOGITS
    assert cases.rel_l2(step, ref[:, T:]) <= REL_LOGITS
    # greedy token: identical whenever the oracle's two best logits are further apart than the logits differ
    top2 = ref[0, T].float().topk(2).values
    if float(top2[0] - top2[1]) > 2 * float((step[0, 0].float() - ref[0, T].float()).abs().max()):
        assert int(step[0, 0].argmax()) == int(ref[0, T].argmax())
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


def test_graph_wrapper_generate_matches_eager(dev, tmp_path):
    from glorcq_b200 import synthetic
    from glorcq_b200.graph_wrapper import GLoRCQGraphWrapper, run_speed_benchmark
    from glorcq_b200.model_builder import load_glorcq_model
    synthetic.write_checkpoint(str(tmp_path), CFG, seed=41, rank=16, attn_rank=32, n_clusters=3)
    model = load_glorcq_model(str(tmp_path), device="cuda:0")
    ids = torch.randint(0, 512, (1, 9), generator=torch.Generator().manual_seed(4)).to(dev)
    eager = model.generate(ids, max_new_tokens=8)
    w = GLoRCQGraphWrapper(model, max_batch_size=1, max_seq_len=32)
    out, seconds = w.generate(ids, max_new_tokens=8)          # captures on first use
    assert out.shape == (1, 17) and seconds > 0
    assert torch.equal(out, eager)
    out2, _ = w.generate(ids, max_new_tokens=8)               # replay of the captured graph only
    assert torch.equal(out2, eager)
    assert w.static_input_ids.shape == (1, 1) and w.static_cache_position.shape == (1,)
    assert w.static_logits.shape == (1, 1, 512)
    r = run_speed_benchmark(model, max_seq_len=32, gen_len=6, input_ids=ids)
    assert set(r) == {"standard_tps", "graph_tps", "speedup"} and r["graph_tps"] > 0
    with pytest.raises(AssertionError):
        w.generate(torch.cat([ids, ids]), max_new_tokens=2)
