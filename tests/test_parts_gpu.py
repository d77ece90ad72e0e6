"""Each part of a layer alone against its plain formula, built through the part registry with
sizes that are not the engine's, and the run order as data (a layer named twice, a layer that reads
another layer's cache)."""
import math

import pytest
import torch

import plain_llama as pl
from helpers import close

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def rt_for(dt):
    from mini_inference_engine_b200.parts import Runtime
    return Runtime(DEV, dt)


def ctx_for(rows, page, tables, num_groups=1):
    from mini_inference_engine_b200.engine.batch import BatchBuilder, BatchRow
    b = BatchBuilder(num_groups, page, DEV)
    return b.build([BatchRow(toks, pos0, [tbl] * num_groups, i + 1, want) for i, (toks, pos0, tbl, want) in enumerate(rows)])


def bound(part, rt, seed=0, dtype=None):
    torch.manual_seed(seed)
    tensors = {}
    for name, spec in part.tensor_specs().items():
        t = torch.randn(spec.shape) * (0.3 if len(spec.shape) > 1 else 1.0)
        tensors[name] = t.to(dtype or rt.dtype)
    part.bind(tensors, rt)
    return {k: v.float() for k, v in tensors.items()}


@pytest.mark.parametrize("dt", DTYPES)
def test_rmsnorm_part(dt):
    from mini_inference_engine_b200.config import PartSpec
    from mini_inference_engine_b200.parts import build_part
    rt = rt_for(dt)
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=72, eps=3e-4)))
    W = bound(norm, rt, 1)
    res = torch.randn(5, 72, device=DEV)
    delta = torch.randn(5, 72).to(dt).to(DEV)
    want = pl.rmsnorm(res.cpu() + delta.float().cpu(), W["weight"], 3e-4)
    close(norm(delta, res), want, dt, "norm part")


@pytest.mark.parametrize("dt", DTYPES)
def test_swiglu_part(dt):
    from mini_inference_engine_b200.config import PartSpec
    from mini_inference_engine_b200.parts import build_part
    rt = rt_for(dt)
    ff = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=40, intermediate_size=56)))
    W = bound(ff, rt, 2)
    x = torch.randn(9, 40).to(dt)
    rnd = pl.round_bf16 if dt == torch.bfloat16 else pl.identity
    want = pl.feed_forward(x.float(), {"p." + k: v for k, v in W.items()}, "p.", rnd)
    close(ff.forward(x.to(DEV), None), want, dt, "swiglu part")


@pytest.mark.parametrize("dt", DTYPES)
def test_embedding_and_tied_head(dt):
    from mini_inference_engine_b200.config import PartSpec
    from mini_inference_engine_b200.parts import build_part
    rt = rt_for(dt)
    emb = build_part("embedding", PartSpec("embedding", dict(vocab_size=50, hidden_size=24)))
    W = bound(emb, rt, 3)
    head = build_part("head", PartSpec("linear_head", dict(vocab_size=50, hidden_size=24, tied=True)))
    head.bind({}, rt, shared=emb.weight)
    ctx = ctx_for([([3, 49, 0], 0, [1], [])], 16, None)
    assert torch.equal(emb.forward(ctx).cpu(), W["weight"][[3, 49, 0]])
    x = torch.randn(4, 24).to(dt)
    logits = head.forward(x.to(DEV))
    assert logits.dtype == torch.float32
    close(logits, pl.linear(x.float(), W["weight"]), dt, "tied head")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,Hkv,D,rot,window", [(4, 2, 16, 16, None), (3, 1, 32, 32, None), (2, 2, 48, 16, 6)])
def test_attention_part_whole_and_cut(dt, H, Hkv, D, rot, window):
    """The attention part on a whole sequence, then the same sequence cut into a portion and single
    tokens on other pages: both must equal the plain layer."""
    from mini_inference_engine_b200.config import PartSpec
    from mini_inference_engine_b200.parts import LayerCache, build_part
    rt = rt_for(dt)
    hidden, T, page, theta = 40, 37, 16, 12345.0
    att = build_part("mixer", PartSpec("attention", dict(
        hidden_size=hidden, num_heads=H, num_kv_heads=Hkv, head_dim=D, window=window,
        position=PartSpec("rope", dict(head_dim=D, rotary_dim=rot, theta=theta, max_position=64)))))
    W = bound(att, rt, H + D)
    x = torch.randn(T, hidden).to(dt)
    rnd = pl.round_bf16 if dt == torch.bfloat16 else pl.identity
    cfg = dict(heads=H, kv_heads=Hkv, head_dim=D, theta=theta, bias=False)
    if rot == D:
        want = pl.attention_layer(x.float(), {"a." + k: v for k, v in W.items()}, "a.", cfg, torch.arange(T), rnd, window)
    else:                                            # partial rotation: the plain layer, rotating the first `rot` dims
        q = rnd(pl.linear(x.float(), W["q_proj.weight"])).view(T, H, D)
        k = rnd(pl.linear(x.float(), W["k_proj.weight"])).view(T, Hkv, D)
        v = rnd(pl.linear(x.float(), W["v_proj.weight"])).view(T, Hkv, D)
        ang = pl.rope_angles(torch.arange(T), rot, theta)
        q = rnd(torch.cat((pl.apply_rope(q[..., :rot], ang), q[..., rot:]), -1))
        k = rnd(torch.cat((pl.apply_rope(k[..., :rot], ang), k[..., rot:]), -1))
        a = rnd(pl.causal_attention(q, k, v, 1 / math.sqrt(D), window))
        want = rnd(pl.linear(a.reshape(T, H * D), W["o_proj.weight"]))
    need = att.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (Hkv, D, window)
    kv = torch.zeros(2, 12, Hkv, page, D, dtype=dt, device=DEV)
    cache = LayerCache(group=0, k=kv[0], v=kv[1], page_size=page)
    tbl = [5, 2, 9]
    got = att.forward(x.to(DEV), ctx_for([(list(range(T)), 0, tbl, [])], page, None), cache)
    close(got, want, dt, "attention part, whole")
    tbl2 = [7, 1, 10]
    got2 = [att.forward(x[:20].to(DEV), ctx_for([([0] * 20, 0, tbl2, [])], page, None), cache)]
    for p in range(20, T):
        got2.append(att.forward(x[p:p + 1].to(DEV), ctx_for([([0], p, tbl2, [])], page, None), cache))
    close(torch.cat(got2, 0), want, dt, "attention part, portion + single tokens")


@pytest.mark.parametrize("dt", DTYPES)
def test_block_part(dt):
    from mini_inference_engine_b200.config import LayerSpec, PartSpec
    from mini_inference_engine_b200.models.decoder import _layer_parts
    from mini_inference_engine_b200.parts import LayerCache
    rt = rt_for(dt)
    h, H, Hkv, D, I, T = 48, 3, 3, 16, 80, 19
    norm = dict(size=h, eps=1e-5)
    ls = LayerSpec("prenorm_residual", dict(
        mixer=PartSpec("attention", dict(hidden_size=h, num_heads=H, num_kv_heads=Hkv, head_dim=D,
                                         position=PartSpec("rope", dict(head_dim=D, rotary_dim=D, theta=1e4, max_position=32))), "a."),
        feed_forward=PartSpec("swiglu", dict(hidden_size=h, intermediate_size=I), "f."),
        mixer_norm=PartSpec("rmsnorm", norm, "n1."), feed_forward_norm=PartSpec("rmsnorm", norm, "n2.")))
    block, named = _layer_parts(ls)
    W = {}
    for i, (prefix, part) in enumerate(named):
        W.update({prefix + k: v for k, v in bound(part, rt, 10 + i).items()})
    res0 = torch.randn(T, h)
    delta0 = torch.randn(T, h).to(dt)
    rnd = pl.round_bf16 if dt == torch.bfloat16 else pl.identity
    cfg = dict(heads=H, kv_heads=Hkv, head_dim=D, theta=1e4, bias=False)
    r = res0 + delta0.float()
    r1 = r + pl.attention_layer(rnd(pl.rmsnorm(r, W["n1.weight"], 1e-5)), W, "a.", cfg, torch.arange(T), rnd)
    want_delta = pl.feed_forward(rnd(pl.rmsnorm(r1, W["n2.weight"], 1e-5)), W, "f.", rnd)
    kv = torch.zeros(2, 6, Hkv, 16, D, dtype=dt, device=DEV)
    res = res0.to(DEV)
    got = block.forward(delta0.to(DEV), res, ctx_for([([0] * T, 0, [3, 4], [])], 16, None),
                        LayerCache(group=0, k=kv[0], v=kv[1], page_size=16))
    close(res, r1, dt, "residual after the mixer")
    close(got, want_delta, dt, "block output")


def test_blocks_that_fold_their_norms_into_the_products():
    """Few tokens in bfloat16 at sizes where the tensor-core product splits K: the mixer and the
    feed-forward take the block's offer, add to the stream in their last product and prepare the next
    norm; the norm then launches nothing and hands the prepared input on.  Two blocks in a row, the
    second told about by the first, against the plain formulas; and the same blocks without the offer."""
    from mini_inference_engine_b200.config import LayerSpec, PartSpec
    from mini_inference_engine_b200.kernels import gemm_tc, ops
    from mini_inference_engine_b200.models.decoder import _layer_parts
    from mini_inference_engine_b200.parts import LayerCache
    from mini_inference_engine_b200.parts.base import StreamUpdated
    dt = torch.bfloat16
    rt = rt_for(dt)
    h, H, Hkv, D, I, T, eps = 512, 8, 2, 64, 1024, 5, 1e-5
    norm = dict(size=h, eps=eps)
    blocks, Ws = [], []
    for b in range(2):
        ls = LayerSpec("prenorm_residual", dict(
            mixer=PartSpec("attention", dict(hidden_size=h, num_heads=H, num_kv_heads=Hkv, head_dim=D,
                                             position=PartSpec("rope", dict(head_dim=D, rotary_dim=D, theta=1e4, max_position=64))), "a."),
            feed_forward=PartSpec("swiglu", dict(hidden_size=h, intermediate_size=I), "f."),
            mixer_norm=PartSpec("rmsnorm", norm, "n1."), feed_forward_norm=PartSpec("rmsnorm", norm, "n2.")))
        block, named = _layer_parts(ls)
        W = {}
        for i, (prefix, part) in enumerate(named):
            torch.manual_seed(100 * b + i)
            tensors = {n: (torch.randn(sp.shape) * (0.04 if len(sp.shape) > 1 else 1.0)).to(dt) for n, sp in part.tensor_specs().items()}
            part.bind(tensors, rt)
            W.update({prefix + k: v.float() for k, v in tensors.items()})
        blocks.append(block)
        Ws.append(W)
    assert blocks[0].mixer.defers_norm(T) and blocks[0].feed_forward.defers_norm(T)
    res0, delta0 = torch.randn(T, h), torch.randn(T, h).to(dt)
    cfg = dict(heads=H, kv_heads=Hkv, head_dim=D, theta=1e4, bias=False)
    r = res0 + delta0.float()
    for W in Ws:                                                  # the plain formulas, two layers
        r = r + pl.attention_layer(pl.round_bf16(pl.rmsnorm(r, W["n1.weight"], eps)), W, "a.", cfg, torch.arange(T), pl.round_bf16)
        last_delta = pl.feed_forward(pl.round_bf16(pl.rmsnorm(r, W["n2.weight"], eps)), W, "f.", pl.round_bf16)
        r_before_ff = r
        r = r + last_delta

    def run(tell_next):
        kv = torch.zeros(2, 2, 6, Hkv, 16, D, dtype=dt, device=DEV)
        res = res0.to(DEV)
        ctx = ctx_for([([0] * T, 0, [3, 4], [])], 16, None)
        before = ops.launches
        d = blocks[0].forward(delta0.to(DEV), res, ctx, LayerCache(group=0, k=kv[0, 0], v=kv[0, 1], page_size=16),
                              **({"next_block": blocks[1]} if tell_next else {}))
        mid = d
        d = blocks[1].forward(d, res, ctx, LayerCache(group=0, k=kv[1, 0], v=kv[1, 1], page_size=16))
        torch.cuda.synchronize()
        gemm_tc.check_error()
        return mid, d, res, ops.launches - before

    mid, d, res, launches = run(True)
    assert isinstance(mid, StreamUpdated) and mid.norm is blocks[1].mixer_norm and mid.deferred is not None
    close(d, last_delta, dt, "output of the second block")       # the last block has nobody to prepare for
    close(res, r_before_ff, dt, "stream after three folded sums")
    mid2, d2, res2, launches2 = run(False)
    assert isinstance(mid2, torch.Tensor)
    close(d2, last_delta, dt, "output without telling the first block about the second")
    close(res2, r_before_ff, dt, "stream without it")
    # folded: norm, q|k|v, attention, out, gate/up, down + q|k|v, attention, out, gate/up, down; the
    # untold first block ends with a plain product and the second starts with a norm kernel
    assert launches == 11 and launches2 == 12


def test_run_order_is_data_a_layer_twice_and_a_shared_cache(tmp_path):
    """A model whose run order names layer 0 twice (own cache each time) and lets layer 1 read the
    cache that the first run of layer 0 wrote.  Whole sequence == portion + single tokens."""
    from mini_inference_engine_b200.config import RunEntry, load_config
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.models.decoder import DecoderModel, expected_tensors
    from mini_inference_engine_b200.weights import random_state
    import dataclasses
    cfg = load_config(dict(vocab_size=100, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                           num_attention_heads=2, num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-5,
                           max_position_embeddings=64, architectures=["LlamaForCausalLM"]))
    spec = dataclasses.replace(cfg.model_spec(), run_order=(RunEntry(0, 0), RunEntry(1, 0, False), RunEntry(0, 1)))
    state = random_state(expected_tensors(spec), 3, torch.float32)
    state = {k: v * (10 if "proj" in k else 1) for k, v in state.items()}     # so that attention matters
    toks = list(range(5, 45))

    def run(cuts):
        model = DecoderModel(spec, state, rt_for(torch.float32))
        assert len(model.cache_layout.kv) == 2            # two caches for three runs
        runner = ModelRunner(model, 9, 16, 2)
        rc, out, p = RequestCache(), [], 0
        for n in cuts:
            out.append(runner.run([(rc, toks[p:p + n], range(n))]))
            p += n
        return torch.cat(out, 0)

    whole = run([40])
    cut = run([23] + [1] * 17)
    close(cut, whole, torch.float32, "run order: cut vs whole")
    # and the shared cache is really read: the same model with layer 1 on a cache of its own differs
    spec2 = dataclasses.replace(spec, run_order=(RunEntry(0, 0), RunEntry(1, 2), RunEntry(0, 1)))
    model2 = DecoderModel(spec2, state, rt_for(torch.float32))
    runner2 = ModelRunner(model2, 9, 16, 2)
    other = runner2.run([(RequestCache(), toks, range(40))])
    assert (other - whole).abs().max() > 1e-3
