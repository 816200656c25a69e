"""Each part of a layer alone on the GPU against its plain counterpart: norm, position table,
feed-forward, attention mixer (with a cache of its own), a whole block."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as pq
import tiny_models as tm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-6, "bfloat16": 1e-2}


def close(a, b, tol):
    a, b = a.double().cpu(), b.double().cpu()
    err, scale = float((a - b).abs().max()), max(1.0, float(b.abs().max()))
    assert err <= tol * scale, f"max error {err:.3e} > {tol * scale:.3e}"


def one_request_batch(cache, n_tokens, past, slot):
    """A StepBatch for one request feeding n_tokens after `past` cached ones."""
    from litellmengine_b200.engine.batch import StepBuffers, StepEntry, pack_step
    buf = StepBuffers(256, 4, len(cache.groups), DEV)
    e = StepEntry(slot, [0] * n_tokens, [])
    e.past = past
    cache.ensure(slot, past + n_tokens)
    batch = pack_step(buf, [e], cache.drain_updates())
    for g, grp in enumerate(cache.groups):
        n = int(buf.host_view("counts")[8 + g])
        if n:
            from litellmengine_b200.csrc import ops
            ops.scatter_int32(grp.table_dev, buf.dev_view(f"upd_index{g}", n), buf.dev_view(f"upd_value{g}", n),
                              buf.dev_view("counts")[8 + g:9 + g], n, buf.status)
    return batch, buf


def test_rmsnorm_part_and_rope_table():
    from litellmengine_b200.config import NormSpec, PositionSpec
    from litellmengine_b200.parts import lookup
    n = lookup("norm", "rmsnorm")(NormSpec("rmsnorm", 2e-5), 100)
    assert n.parameters()["weight"].shape == (100,) and n.parameters()["weight"].role == "scale"
    w = 1 + 0.1 * torch.randn(100)
    n.load({"weight": w.to(DEV)})
    x = torch.randn(9, 100)
    close(n.forward(x.to(DEV), torch.float32), pq.rms_norm(x, w, 2e-5), 1e-6)
    for theta, d in ((10000.0, 16), (1e6, 128), (50000.0, 48)):
        r = lookup("position", "rope")(PositionSpec("rope", theta=theta, rotary_dim=d), d, DEV)
        assert torch.equal(r.inv_freq.cpu(), pq.rope_inv_freq(d, theta)) and r.rotary_dim == d
    with pytest.raises(ValueError):
        lookup("position", "rope")(PositionSpec("rope", theta=1e4, rotary_dim=18), 16, DEV)
    with pytest.raises(KeyError, match="registered"):
        lookup("norm", "layernorm")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part(dtype):
    from litellmengine_b200.config import FeedForwardSpec
    from litellmengine_b200.parts import lookup
    torch.manual_seed(0)
    H, I = 72, 200
    ff = lookup("feed_forward", "swiglu")(FeedForwardSpec("swiglu", intermediate_size=I), H, DT[dtype], DEV)
    assert {k: v.shape for k, v in ff.parameters().items()} == {
        "gate_proj.weight": (I, H), "up_proj.weight": (I, H), "down_proj.weight": (H, I)}
    w = {k: (torch.randn(v.shape) * 0.1).to(DT[dtype]) for k, v in ff.parameters().items()}
    ff.load({k: v.to(DEV) for k, v in w.items()})
    x = torch.randn(21, H).to(DT[dtype])
    act = pq.to_bf16 if dtype == "bfloat16" else pq.identity
    ref = pq.swiglu(x.float(), {f"m.{k}": v.float() for k, v in w.items()}, "m", act=act)
    close(ff.forward(x.to(DEV)), ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,window", [(6, 2, 48, None), (4, 4, 16, 7), (8, 1, 64, None)])
def test_attention_mixer_alone_in_two_portions(dtype, nq, nkv, d, window):
    from litellmengine_b200.cache import CacheManager
    from litellmengine_b200.config import MixerSpec, NormSpec, PositionSpec
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.parts import StageContext, lookup
    ops.configure_library_products()
    torch.manual_seed(1)
    H, T, page, eps, theta = 88, 45, 8, 1e-5, 30000.0
    spec = MixerSpec(kind="attention", num_heads=nq, num_kv_heads=nkv, head_dim=d, qk_norm=NormSpec("rmsnorm", eps),
                     position=PositionSpec("rope", theta=theta, rotary_dim=d), window=window)
    mixer = lookup("mixer", "attention")(spec, H, DT[dtype], DEV)
    bf = dtype == "bfloat16"
    w = {}
    for k, p in mixer.parameters().items():
        t = 1 + 0.1 * torch.randn(p.shape) if p.role == "scale" else torch.randn(p.shape) * 0.15
        w[k] = t.to(torch.bfloat16).float() if bf else t
    mixer.load({k: (v.to(DT[dtype]) if v.dim() == 2 else v).to(DEV) for k, v in w.items()})
    cache = CacheManager([mixer.cache_need()], page, 64, 2, dtype=DT[dtype], device=DEV)
    slot = cache.admit()
    x = torch.randn(T, H)
    x = x.to(torch.bfloat16).float() if bf else x
    outs = []
    for lo, hi in ((0, 29), (29, T)):                      # a portion from zero, then one at past 29
        batch, buf = one_request_batch(cache, hi - lo, lo, slot)
        kv, table, _ = cache.stage_cache(0)
        ctx = StageContext(batch=batch, stage=0, cache=kv, block_table=table, page_size=page, writes_cache=True,
                           state=None, status=buf.status)
        outs.append(mixer.forward(x[lo:hi].to(DT[dtype]).to(DEV), ctx))
        cache.commit(slot, hi)
        assert buf.status.tolist() == [0, 0]
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, rms_norm_eps=eps, rope_theta=theta)
    act = pq.to_bf16 if bf else pq.identity
    ref = pq.attention_block(x, torch.arange(T, dtype=torch.int32), {f"a.{k}": v for k, v in w.items()}, "a", cfg,
                             window=window, act=act)
    close(torch.cat(outs), ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_block_alone(dtype):
    from litellmengine_b200.cache import CacheManager
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.parts import Block, StageContext
    ops.configure_library_products()
    cfg = tm.TINY_C
    plan = config_from_dict(cfg).plan()
    block = Block(plan.blocks[1], plan.hidden_size, DT[dtype], DEV)
    bf = dtype == "bfloat16"
    allw = tm.make_weights(cfg, 3, bf16_exact=bf)
    names = {k: f"model.layers.1.{k}" for k in block.parameters()}
    block.load({k: (allw[n].to(DT[dtype]) if allw[n].dim() == 2 else allw[n]).to(DEV) for k, n in names.items()})
    cache = CacheManager([block.mixer.cache_need()], 16, 64, 1, dtype=DT[dtype], device=DEV)
    slot = cache.admit()
    T = 40
    torch.manual_seed(2)
    h = torch.randn(T, plan.hidden_size)
    pending = torch.randn(T, plan.hidden_size) * 0.1        # the previous layer's unadded output
    batch, buf = one_request_batch(cache, T, 0, slot)
    kv, table, _ = cache.stage_cache(0)
    ctx = StageContext(batch=batch, stage=0, cache=kv, block_table=table, page_size=16, writes_cache=True, state=None,
                       status=buf.status)
    hg = h.to(DEV)
    hg, delta = block.forward(hg, pending.to(DEV), ctx)
    act = pq.to_bf16 if bf else pq.identity
    ref = pq.decoder_layer(h + pending, torch.arange(T, dtype=torch.int32), allw, 1, cfg, act=act)
    close(hg + delta.float(), ref, TOL[dtype])


def test_random_weights_do_not_depend_on_where_they_are_drawn():
    """The random-weights mode draws a tensor as a function of (seed, name, element): on the host and on
    the GPU the same bits, in float32 and after rounding to bfloat16, for shapes past one chunk of the
    generator too."""
    from litellmengine_b200.weights import ParamSpec, RandomSource
    from litellmengine_b200.weights.loader import seeded_normal
    params = {"a.weight": ParamSpec((300, 129)), "n.weight": ParamSpec((77,), role="scale", init=("one_plus_normal", 0.01))}
    for dtype in (torch.float32, torch.bfloat16):
        host, dev = RandomSource(params, 9, dtype, "cpu"), RandomSource(params, 9, dtype, DEV)
        for name in params:
            assert torch.equal(host.get(name), dev.get(name).cpu()), name
    a = seeded_normal((5000, 700), 123456789, 0.02, 0.0, "cpu", chunk=1 << 20)
    b = seeded_normal((5000, 700), 123456789, 0.02, 0.0, DEV)
    assert torch.equal(a, b.cpu()) and abs(float(a.std()) - 0.02) < 2e-4 and abs(float(a.mean())) < 1e-4
