"""The framework's generality, shown with toy parts that exist only in this file: a mixer with
a state of its own (no pages), a windowed attention layer (a cache group that gives pages
back), a layer that runs twice, and a layer that reads another stage's cache.  They are
registered, built and stepped here without a change to the framework's files, in every way of
cutting, against plain code.  None of this is a model of anyone's."""
from dataclasses import dataclass
from typing import Dict

import numpy as np
import pytest
import torch

import plain_qwen3 as pq
import replay_helpers as rh

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

H, NQ, NKV, D, INTER, VOCAB, WINDOW, EPS, THETA = 48, 4, 2, 16, 80, 97, 6, 1e-5, 10000.0
PCFG = dict(num_attention_heads=NQ, num_key_value_heads=NKV, head_dim=D, rms_norm_eps=EPS, rope_theta=THETA)


def register_toys():
    from litellmengine_b200.cache import StateNeed
    from litellmengine_b200.config import (BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec,
                                           StageSpec, register_architecture)
    from litellmengine_b200.parts import register_mixer
    from litellmengine_b200.weights import ParamSpec

    @register_mixer("toy_running_mean")
    class RunningMean:
        """out[t] = W . mean(x[0..t]); the state per request is the running sum and the count."""

        def __init__(self, spec, hidden_size, compute_dtype, device):
            self.hidden, self.dtype = hidden_size, compute_dtype
            self.w = None

        def parameters(self) -> Dict[str, ParamSpec]:
            return {"mix.weight": ParamSpec((self.hidden, self.hidden))}

        def load(self, t):
            self.w = t["mix.weight"].float()

        def cache_need(self):
            return StateNeed((self.hidden + 1,), "float32")

        def forward(self, x, ctx):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            row = 0
            for e in ctx.batch.entries:
                n = len(e.tokens)
                st = ctx.state[e.slot]
                assert int(st[-1].item()) == e.past, "the slot's state does not belong to this request"
                sums = st[:-1] + torch.cumsum(x[row:row + n].float(), dim=0)
                counts = st[-1] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[row:row + n] = (sums / counts[:, None]) @ self.w.T
                st[:-1] = sums[-1]
                st[-1] = counts[-1]
                row += n
            return out

    @register_architecture("ToyPartsForCausalLM")
    @dataclass(frozen=True)
    class ToyConfig:
        layers: int = 3

        @classmethod
        def from_dict(cls, d):
            return cls()

        def to_dict(self):
            return {"architectures": ["ToyPartsForCausalLM"]}

        def plan(self):
            norm = NormSpec("rmsnorm", EPS)
            rope = PositionSpec("rope", theta=THETA, rotary_dim=D)
            ffn = FeedForwardSpec("swiglu", intermediate_size=INTER)
            windowed = MixerSpec("attention", NQ, NKV, D, qk_norm=norm, position=rope, window=WINDOW)
            full = MixerSpec("attention", NQ, NKV, D, qk_norm=norm, position=rope)
            reader = MixerSpec("attention", NQ, NKV, D, qk_norm=norm, position=rope, has_kv=False)
            blocks = (
                BlockSpec("pre_norm", windowed, ffn, norm, norm, weight_prefix="toy.0"),
                BlockSpec("pre_norm", MixerSpec("toy_running_mean", weight_prefix="mean"), ffn, norm, norm,
                          weight_prefix="toy.1"),
                BlockSpec("pre_norm", full, ffn, norm, norm, weight_prefix="toy.2"),
                BlockSpec("pre_norm", reader, ffn, norm, norm, weight_prefix="toy.3"),
            )
            # windowed, running mean, full, the windowed layer again (a cache of its own), a reader of
            # stage 2's keys and values, the running mean again (a state of its own)
            order = (StageSpec(0), StageSpec(1), StageSpec(2), StageSpec(0), StageSpec(3, cache_from=2), StageSpec(1))
            return ModelPlan(H, VOCAB, blocks, order, norm, tie_word_embeddings=True, max_position=512,
                             embedding_name="toy.embed", final_norm_name="toy.norm", output_name="toy.head")
    return ToyConfig


def unregister_toys():
    from litellmengine_b200.config import unregister_architecture
    from litellmengine_b200.parts import unregister
    unregister("mixer", "toy_running_mean")
    unregister_architecture("ToyPartsForCausalLM")


def plain_toy_logits(ids, w, act=pq.identity, wd=torch.float32):
    """The same wiring in plain code: whole sequence, no cache, no state."""
    w = {k: v.to(wd) for k, v in w.items()}
    T = len(ids)
    pos = torch.arange(T, dtype=torch.int32)
    h = pq.embedding(torch.as_tensor(ids), w["toy.embed"]).to(wd)

    def ffn_part(h, p):
        y = act(pq.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], EPS))
        return h + pq.swiglu(y, w, f"{p}.mlp", act)

    def attn_layer(h, p, window=None, kv=None):
        x = act(pq.rms_norm(h, w[f"{p}.input_layernorm.weight"], EPS))
        return ffn_part(h + pq.attention_block(x, pos, w, f"{p}.self_attn", PCFG, window=window, act=act, kv=kv), p)

    def mean_layer(h, p):
        x = act(pq.rms_norm(h, w[f"{p}.input_layernorm.weight"], EPS))
        run = torch.cumsum(x, dim=0) / torch.arange(1, T + 1, dtype=wd)[:, None]
        return ffn_part(h + run @ w[f"{p}.mean.mix.weight"].T, p)

    h = attn_layer(h, "toy.0", window=WINDOW)
    h = mean_layer(h, "toy.1")
    x2 = act(pq.rms_norm(h, w["toy.2.input_layernorm.weight"], EPS))
    _, k2, v2 = pq.attention_qkv(x2, pos, w, "toy.2.self_attn", PCFG, act)
    h = attn_layer(h, "toy.2")
    h = attn_layer(h, "toy.0", window=WINDOW)
    h = attn_layer(h, "toy.3", kv=(k2, v2))
    h = mean_layer(h, "toy.1")
    hn = act(pq.rms_norm(h, w["toy.norm"], EPS))
    return (hn @ w["toy.embed"].T).float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(dtype, tmp_path):
    from litellmengine_b200.config import load_config
    from litellmengine_b200.engine import ModelRunner
    from litellmengine_b200.weights import SafetensorsSource, write_random_model
    Toy = register_toys()
    try:
        store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        folder = write_random_model(Toy(), str(tmp_path / "toy"), seed=4, dtype=store)
        assert type(load_config(folder)) is Toy
        src = SafetensorsSource(folder)
        w = {n: src.get(n).float() for n in src.names()}
        assert "toy.3.self_attn.k_proj.weight" not in w and "toy.1.mean.mix.weight" in w and "toy.head" not in w
        w = {k: (v * 4.0 if k.endswith("q_norm.weight") else v) for k, v in w.items()}     # sharpen attention
        rng = np.random.RandomState(0)
        reqs = {f"r{i}": [int(t) for t in rng.randint(0, VOCAB, n)] for i, n in enumerate((3, 40, 71, 18, 55))}
        if dtype == "bfloat16":
            ref = {r: plain_toy_logits(t, w, act=pq.to_bf16).numpy() for r, t in reqs.items()}
        else:
            ref = {r: plain_toy_logits(t, w, wd=torch.float64).numpy() for r, t in reqs.items()}
        from litellmengine_b200.weights import DictSource
        for what, steps in (("whole", rh.trace_whole(reqs)), ("tail", rh.trace_tail_decode(reqs, 32)),
                            ("portions", rh.trace_portions(reqs, 1)), ("mixed", rh.trace_mixed(reqs, 2, 4))):
            runner = ModelRunner.from_config(
                Toy(), dtype=dtype, device=DEV, page_size=4, max_requests=4, max_tokens_per_step=128,
                max_total_tokens=rh.peak_tokens(steps, 4),
                source=DictSource({k: (v.to(store) if v.dim() == 2 else v) for k, v in w.items()}))
            groups = runner.cache.groups
            assert sorted((str(g.need.window), len(g.stages)) for g in groups) == [("6", 2), ("None", 1)]
            assert set(runner.cache.stage_state) == {1, 5} and runner.cache.stage_group[4] == runner.cache.stage_group[2]
            got = rh.run_trace(runner, steps)
            rh.assert_rows_match(got, ref, rh.tol_for(dtype), f"toy {dtype} {what}")
        # the windowed group really gave pages back while a request was still running
        runner = ModelRunner.from_config(Toy(), dtype=dtype, device=DEV, page_size=4, max_requests=2,
                                         max_tokens_per_step=128, max_total_tokens=128,
                                         source=DictSource({k: (v.to(store) if v.dim() == 2 else v) for k, v in w.items()}))
        from litellmengine_b200.engine import StepEntry
        s = runner.admit()
        runner.step([StepEntry(s, reqs["r2"], [])])
        win = [g for g in runner.cache.groups if g.need.window == WINDOW][0]
        full = [g for g in runner.cache.groups if g.need.window is None][0]
        assert len(full.held_pages(s)) == 18 and len(win.held_pages(s)) == 2
        runner.release(s)
    finally:
        unregister_toys()
