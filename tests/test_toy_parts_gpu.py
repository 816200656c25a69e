"""The framework's generality, shown with toy parts that exist only in this file: a mixer with
a state of its own (no pages; updated by tensor operations alone, so its steps are replayed as graphs), a windowed attention layer (a cache group that gives pages
back), a layer that runs twice, a layer that reads another stage's cache, a feed-forward that
routes tokens to experts, and a position encoding with a frequency table of its own.  They are
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

        graph_safe = True          # tensor operations on the current stream only: no host reads, no loops over entries

        def forward(self, x, ctx):
            b = ctx.batch
            T = x.shape[0]
            ent = b.token_entry.long()
            slot = b.entry_slot.long()[ent]                              # [T] the slot of each token's request
            start = b.entry_q_start.long()[ent]                          # [T] first row of the token's entry
            cs = torch.cumsum(x.double(), dim=0)                         # in double: the difference below must not cancel
            before = torch.where((start > 0)[:, None], cs[(start - 1).clamp(min=0)], torch.zeros_like(cs))
            sums = ctx.state[slot, :-1] + (cs - before).float()          # running sum inside the entry, on top of the slot's
            counts = ctx.state[slot, -1] + (torch.arange(T, device=x.device) - start + 1).float()
            last = b.entry_q_start.long() + b.entry_q_len.long() - 1     # each entry's last row carries the new state
            ctx.state[b.entry_slot.long()] = torch.cat([sums[last], counts[last][:, None]], dim=1)
            return (sums / counts[:, None]) @ self.w.T

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
            assert runner.use_graphs                                   # every part of the toy model launches kernels only
            got = rh.run_trace(runner, steps)
            rh.assert_rows_match(got, ref, rh.tol_for(dtype), f"toy {dtype} {what}")
            if what in ("tail", "mixed"):                              # steps of one size recur: they were replayed as graphs,
                assert runner.graph_replays > 0                        # the mixer's state advancing once per step all the same
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


# ---- a feed-forward with routing and another position encoding --------------------------------
E_EXPERTS, E_INTER = 3, 32


def register_routed_toys():
    from litellmengine_b200.config import (BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec,
                                           StageSpec, register_architecture)
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.parts import Rotation, register_feed_forward, register_position
    from litellmengine_b200.weights import ParamSpec

    @register_position("toy_linear_frequencies")
    class LinearFrequencies:
        """A rotation whose frequencies fall off linearly instead of geometrically:
        inv_freq[i] = (1 - i / (rotary_dim / 2)) / theta.  The mixer's kernel only wants the table."""

        def __init__(self, spec, head_dim, device):
            self.rotary_dim = spec.rotary_dim or head_dim
            half = self.rotary_dim // 2
            self.inv_freq = ((1.0 - torch.arange(half, dtype=torch.float32) / half) / spec.theta).to(device)

        def rotation(self, batch):
            return Rotation(self.inv_freq, self.rotary_dim)

    @register_feed_forward("toy_top1_experts")
    class Top1Experts:
        """Each token goes to the expert with the largest router logit (logits in float32, ties to
        the lowest index) and gets that expert's SwiGLU, scaled by the softmax weight of the choice."""

        def __init__(self, spec, hidden_size, compute_dtype, device):
            self.hidden, self.dtype = hidden_size, compute_dtype
            self.inter = spec.intermediate_size
            self.router = self.gate_up = self.down = None

        def parameters(self) -> Dict[str, ParamSpec]:
            out = {"router.weight": ParamSpec((E_EXPERTS, self.hidden))}
            for e in range(E_EXPERTS):
                out[f"experts.{e}.gate_proj.weight"] = ParamSpec((self.inter, self.hidden))
                out[f"experts.{e}.up_proj.weight"] = ParamSpec((self.inter, self.hidden))
                out[f"experts.{e}.down_proj.weight"] = ParamSpec((self.hidden, self.inter))
            return out

        def load(self, t):
            self.router = t["router.weight"].float()
            self.gate_up = [torch.cat([t[f"experts.{e}.gate_proj.weight"], t[f"experts.{e}.up_proj.weight"]]).contiguous()
                            for e in range(E_EXPERTS)]
            self.down = [t[f"experts.{e}.down_proj.weight"].contiguous() for e in range(E_EXPERTS)]

        def forward(self, x, partials_ok=False):
            logits = x.float() @ self.router.T                                   # router logits in 32-bit
            prob = torch.softmax(logits, dim=-1)
            choice = torch.argmax(logits, dim=-1)
            out = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
            for e in range(E_EXPERTS):
                idx = torch.nonzero(choice == e).flatten()
                if idx.numel() == 0:
                    continue
                xe = x[idx].contiguous()
                y = ops.linear(ops.silu_and_mul(ops.linear(xe, self.gate_up[e], out_dtype=self.dtype)), self.down[e],
                               out_dtype=torch.float32)
                out[idx] = y * prob[idx, e][:, None]
            return out

    @register_architecture("ToyRoutedForCausalLM")
    @dataclass(frozen=True)
    class ToyRouted:
        @classmethod
        def from_dict(cls, d):
            return cls()

        def to_dict(self):
            return {"architectures": ["ToyRoutedForCausalLM"]}

        def plan(self):
            norm = NormSpec("rmsnorm", EPS)
            pos = PositionSpec("toy_linear_frequencies", theta=40.0, rotary_dim=D)
            attn = MixerSpec("attention", NQ, NKV, D, qk_norm=norm, position=pos)
            routed = FeedForwardSpec("toy_top1_experts", intermediate_size=E_INTER)
            dense = FeedForwardSpec("swiglu", intermediate_size=INTER)
            blocks = (BlockSpec("pre_norm", attn, routed, norm, norm, weight_prefix="toy.0"),
                      BlockSpec("pre_norm", attn, dense, norm, norm, weight_prefix="toy.1"))
            return ModelPlan(H, VOCAB, blocks, (StageSpec(0), StageSpec(1), StageSpec(0)), norm, tie_word_embeddings=True,
                             max_position=512, embedding_name="toy.embed", final_norm_name="toy.norm",
                             output_name="toy.head")
    return ToyRouted


def plain_routed_logits(ids, w):
    """Plain code for the routed toy, in double precision."""
    w = {k: v.double() for k, v in w.items()}
    T = len(ids)
    pos = torch.arange(T, dtype=torch.float64)
    half = D // 2
    inv = ((1.0 - torch.arange(half, dtype=torch.float32) / half) / torch.tensor(40.0)).double()   # the table is float32
    ang = (pos[:, None].float() * inv.float()[None, :]).double()                                    # and so is the angle

    def rotate(x):                                                     # [T, heads, D]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)

    def attention(x, p):
        q = (x @ w[f"{p}.q_proj.weight"].T).view(T, NQ, D)
        k = (x @ w[f"{p}.k_proj.weight"].T).view(T, NKV, D)
        v = (x @ w[f"{p}.v_proj.weight"].T).view(T, NKV, D)
        q = rotate(pq.rms_norm(q, w[f"{p}.q_norm.weight"], EPS))
        k = rotate(pq.rms_norm(k, w[f"{p}.k_norm.weight"], EPS))
        return pq.causal_attention(q, k, v).reshape(T, -1) @ w[f"{p}.o_proj.weight"].T

    def routed(y, p):
        logits = y @ w[f"{p}.router.weight"].T
        prob = torch.softmax(logits, dim=-1)
        choice = torch.argmax(logits, dim=-1)
        out = torch.zeros_like(y)
        for t in range(T):
            e = int(choice[t])
            out[t] = pq.swiglu(y[t:t + 1], w, f"{p}.experts.{e}")[0] * prob[t, e]
        return out

    h = pq.embedding(torch.as_tensor(ids), w["toy.embed"]).double()
    for p, ffn in (("toy.0", "routed"), ("toy.1", "dense"), ("toy.0", "routed")):
        h = h + attention(pq.rms_norm(h, w[f"{p}.input_layernorm.weight"], EPS), f"{p}.self_attn")
        y = pq.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], EPS)
        h = h + (routed(y, f"{p}.mlp") if ffn == "routed" else pq.swiglu(y, w, f"{p}.mlp"))
    return (pq.rms_norm(h, w["toy.norm"], EPS) @ w["toy.embed"].T).float()


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """A feed-forward that routes each token to one of three experts and a position encoding with a
    frequency table of its own, registered here, beside the framework's attention and dense
    feed-forward, in a model whose first layer runs twice.  Float32 (a routing decision is a
    discontinuity: under bfloat16 rounding a near-tie may fall the other way)."""
    from litellmengine_b200.config import unregister_architecture
    from litellmengine_b200.engine import ModelRunner
    from litellmengine_b200.parts import unregister
    from litellmengine_b200.weights import DictSource, SafetensorsSource, write_random_model
    Toy = register_routed_toys()
    try:
        folder = write_random_model(Toy(), str(tmp_path / "routed"), seed=9, dtype=torch.float32)
        src = SafetensorsSource(folder)
        w = {n: src.get(n).float() for n in src.names()}
        assert "toy.0.mlp.experts.2.down_proj.weight" in w and "toy.1.mlp.gate_proj.weight" in w
        w = {k: (v * 4.0 if k.endswith("q_norm.weight") else v * 30.0 if k.endswith("router.weight") else v)
             for k, v in w.items()}                                    # sharp attention, decided routing
        rng = np.random.RandomState(1)
        reqs = {f"r{i}": [int(t) for t in rng.randint(0, VOCAB, n)] for i, n in enumerate((2, 37, 64, 21))}
        ref = {r: plain_routed_logits(t, w).numpy() for r, t in reqs.items()}
        used = set()
        for t in reqs.values():                                        # the test is about routing: all experts must get tokens
            y = pq.rms_norm(pq.embedding(torch.as_tensor(t), w["toy.embed"]).float(), w["toy.0.post_attention_layernorm.weight"], EPS)
            used |= set(torch.argmax(y @ w["toy.0.mlp.router.weight"].T, dim=-1).tolist())
        assert used == {0, 1, 2}
        for what, steps in (("whole", rh.trace_whole(reqs)), ("tail", rh.trace_tail_decode(reqs, 32)),
                            ("portions", rh.trace_portions(reqs, 1)), ("mixed", rh.trace_mixed(reqs, 2, 4))):
            runner = ModelRunner.from_config(Toy(), dtype="float32", device=DEV, page_size=4, max_requests=4,
                                             max_tokens_per_step=128, max_total_tokens=rh.peak_tokens(steps, 4),
                                             source=DictSource(dict(w)))
            assert not runner.use_graphs                               # the routed part reads its choices on the host
            got = rh.run_trace(runner, steps)
            rh.assert_rows_match(got, ref, rh.FP32_TOL, f"routed toy {what}")
    finally:
        unregister("feed_forward", "toy_top1_experts")
        unregister("position", "toy_linear_frequencies")
        unregister_architecture("ToyRoutedForCausalLM")


# ---- a position encoding that is no rotation, and a mixer whose keys and values differ in width ----
DK, DV = 16, 8


def register_offset_toys():
    from litellmengine_b200.cache import PagedNeed
    from litellmengine_b200.config import (BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec,
                                           StageSpec, register_architecture)
    from litellmengine_b200.parts import register_mixer, register_position
    from litellmengine_b200.weights import ParamSpec

    @register_position("toy_offsets")
    class Offsets:
        """q += A[position], k += B[position] with fixed tables: an encoding by absolute position that
        is not a rotation, so it has `apply` and no `rotation`."""

        def __init__(self, spec, head_dim, device):
            a, b = offset_tables(head_dim)
            self.a, self.b = a.to(device), b.to(device)

        def apply(self, q, k, batch):
            pos = batch.positions.long()
            return q + self.a[pos][:, None, :], (k + self.b[pos][:, None, :]) if k is not None else None

    @register_mixer("toy_narrow_values")
    class NarrowValues:
        """Causal attention without any position encoding whose keys are DK wide and whose values are
        DV wide: its pages hold two tensors of different widths."""

        def __init__(self, spec, hidden_size, compute_dtype, device):
            self.hidden = hidden_size
            self.w = {}

        def parameters(self) -> Dict[str, ParamSpec]:
            return {"q_proj.weight": ParamSpec((NQ * DK, self.hidden)), "k_proj.weight": ParamSpec((NKV * DK, self.hidden)),
                    "v_proj.weight": ParamSpec((NKV * DV, self.hidden)), "o_proj.weight": ParamSpec((self.hidden, NQ * DV))}

        def load(self, t):
            self.w = {k: v.float() for k, v in t.items()}

        def cache_need(self):
            return PagedNeed(NKV, DK, None, value_dim=DV)

        def forward(self, x, ctx):
            b, P = ctx.batch, ctx.page_size
            assert ctx.cache is None and ctx.cache_keys.shape[-1] == DK and ctx.cache_values.shape[-1] == DV
            T = x.shape[0]
            xf = x.float()
            q = (xf @ self.w["q_proj.weight"].T).view(T, NQ, DK)
            k = (xf @ self.w["k_proj.weight"].T).view(T, NKV, DK)
            v = (xf @ self.w["v_proj.weight"].T).view(T, NKV, DV)
            pos = b.positions.long()
            slot = b.entry_slot.long()[b.token_entry.long()]
            page = ctx.block_table.long()[slot, pos // P]
            ctx.cache_keys[page, :, pos % P, :] = k.to(ctx.cache_keys.dtype)
            ctx.cache_values[page, :, pos % P, :] = v.to(ctx.cache_values.dtype)
            out = torch.empty((T, NQ, DV), dtype=torch.float32, device=x.device)
            row = 0
            for e in b.entries:
                n, kv_len = len(e.tokens), e.past + len(e.tokens)
                pages = ctx.block_table[e.slot, :(kv_len + P - 1) // P].long()
                keys = ctx.cache_keys[pages].permute(0, 2, 1, 3).reshape(-1, NKV, DK)[:kv_len].float()
                vals = ctx.cache_values[pages].permute(0, 2, 1, 3).reshape(-1, NKV, DV)[:kv_len].float()
                seen = torch.arange(kv_len, device=x.device)[None, :] <= (e.past + torch.arange(n, device=x.device))[:, None]
                for h in range(NQ):
                    s = (q[row:row + n, h] @ keys[:, h // (NQ // NKV)].T) / (DK ** 0.5)
                    out[row:row + n, h] = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1) @ vals[:, h // (NQ // NKV)]
                row += n
            return out.view(T, NQ * DV) @ self.w["o_proj.weight"].T

    @register_architecture("ToyOffsetsForCausalLM")
    @dataclass(frozen=True)
    class ToyOffsets:
        @classmethod
        def from_dict(cls, d):
            return cls()

        def to_dict(self):
            return {"architectures": ["ToyOffsetsForCausalLM"]}

        def plan(self):
            norm = NormSpec("rmsnorm", EPS)
            attn = MixerSpec("attention", NQ, NKV, D, qk_norm=norm, position=PositionSpec("toy_offsets"))
            ffn = FeedForwardSpec("swiglu", intermediate_size=INTER)
            blocks = (BlockSpec("pre_norm", attn, ffn, norm, norm, weight_prefix="toy.0"),
                      BlockSpec("pre_norm", MixerSpec("toy_narrow_values", weight_prefix="narrow"), ffn, norm, norm,
                                weight_prefix="toy.1"))
            return ModelPlan(H, VOCAB, blocks, (StageSpec(0), StageSpec(1), StageSpec(0)), norm, tie_word_embeddings=True,
                             max_position=512, embedding_name="toy.embed", final_norm_name="toy.norm",
                             output_name="toy.head")
    return ToyOffsets


def offset_tables(head_dim, positions=512):
    p = torch.arange(positions, dtype=torch.float32)[:, None]
    i = torch.arange(head_dim, dtype=torch.float32)[None, :]
    return 0.5 * torch.sin(0.37 * p + i), 0.5 * torch.cos(0.11 * p * (i + 1.0))


def plain_offsets_logits(ids, w, act=pq.identity, wd=torch.float32):
    """Plain code for the offsets toy: whole sequence, no cache."""
    w = {k: v.to(wd) for k, v in w.items()}
    T = len(ids)
    a, b = (t[:T].to(wd) for t in offset_tables(D))

    def offset_attention(x, p):
        q = pq.rms_norm((x @ w[f"{p}.q_proj.weight"].T).view(T, NQ, D), w[f"{p}.q_norm.weight"], EPS)
        k = pq.rms_norm((x @ w[f"{p}.k_proj.weight"].T).view(T, NKV, D), w[f"{p}.k_norm.weight"], EPS)
        v = (x @ w[f"{p}.v_proj.weight"].T).view(T, NKV, D)
        q, k = act(q + a[:, None, :]), act(k + b[:, None, :])
        return act(pq.causal_attention(q, k, act(v))).reshape(T, -1) @ w[f"{p}.o_proj.weight"].T

    def narrow_attention(x, p):
        q = (x @ w[f"{p}.q_proj.weight"].T).view(T, NQ, DK)
        k = act((x @ w[f"{p}.k_proj.weight"].T).view(T, NKV, DK))
        v = act((x @ w[f"{p}.v_proj.weight"].T).view(T, NKV, DV))
        out = torch.empty((T, NQ, DV), dtype=wd)
        seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
        for h in range(NQ):
            s = (q[:, h] @ k[:, h // (NQ // NKV)].T) / (DK ** 0.5)
            out[:, h] = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1) @ v[:, h // (NQ // NKV)]
        return out.reshape(T, -1) @ w[f"{p}.o_proj.weight"].T

    h = pq.embedding(torch.as_tensor(ids), w["toy.embed"]).to(wd)
    for p, kind in (("toy.0", "offsets"), ("toy.1", "narrow"), ("toy.0", "offsets")):
        x = act(pq.rms_norm(h, w[f"{p}.input_layernorm.weight"], EPS))
        h = h + (offset_attention(x, f"{p}.self_attn") if kind == "offsets" else narrow_attention(x, f"{p}.narrow"))
        y = act(pq.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], EPS))
        h = h + pq.swiglu(y, w, f"{p}.mlp", act)
    return (act(pq.rms_norm(h, w["toy.norm"], EPS)) @ w["toy.embed"].T).float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_that_is_no_rotation_and_a_mixer_with_narrow_values(dtype, tmp_path):
    """A position part with `apply` instead of `rotation` (the attention mixer then runs its norms,
    the part, and the cache write as separate kernels), and a mixer that asks for pages whose keys
    and values differ in width.  Both are registered here; nothing in the package names them."""
    from litellmengine_b200.config import unregister_architecture
    from litellmengine_b200.engine import ModelRunner
    from litellmengine_b200.parts import unregister
    from litellmengine_b200.weights import DictSource, SafetensorsSource, write_random_model
    Toy = register_offset_toys()
    try:
        store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        folder = write_random_model(Toy(), str(tmp_path / "offsets"), seed=11, dtype=store)
        src = SafetensorsSource(folder)
        w = {n: src.get(n).float() for n in src.names()}
        assert w["toy.1.narrow.v_proj.weight"].shape == (NKV * DV, H) and w["toy.1.narrow.o_proj.weight"].shape == (H, NQ * DV)
        w = {k: (v * 4.0 if k.endswith("q_norm.weight") else v * 8.0 if "narrow.q_proj" in k else v) for k, v in w.items()}
        rng = np.random.RandomState(3)
        reqs = {f"r{i}": [int(t) for t in rng.randint(0, VOCAB, n)] for i, n in enumerate((2, 45, 70, 19, 33))}
        if dtype == "bfloat16":
            ref = {r: plain_offsets_logits(t, w, act=pq.to_bf16).numpy() for r, t in reqs.items()}
        else:
            ref = {r: plain_offsets_logits(t, w, wd=torch.float64).numpy() for r, t in reqs.items()}
        for what, steps in (("whole", rh.trace_whole(reqs)), ("tail", rh.trace_tail_decode(reqs, 32)),
                            ("portions", rh.trace_portions(reqs, 1)), ("mixed", rh.trace_mixed(reqs, 2, 4))):
            runner = ModelRunner.from_config(
                Toy(), dtype=dtype, device=DEV, page_size=4, max_requests=4, max_tokens_per_step=128,
                max_total_tokens=rh.peak_tokens(steps, 4),
                source=DictSource({k: (v.to(store) if v.dim() == 2 else v) for k, v in w.items()}))
            widths = sorted((g.need.key_width, g.need.value_width, len(g.stages)) for g in runner.cache.groups)
            assert widths == [(DK, DV, 1), (D, D, 2)]
            narrow = [g for g in runner.cache.groups if g.need.value_width == DV][0]
            assert narrow.kv is None and narrow.keys.shape[-1] == DK and narrow.values.shape[-1] == DV
            assert runner.cache.bytes_per_token() == (2 * NKV * 2 * D + NKV * (DK + DV)) * (2 if dtype == "bfloat16" else 4)
            got = rh.run_trace(runner, steps)
            rh.assert_rows_match(got, ref, rh.tol_for(dtype), f"offsets toy {dtype} {what}")
    finally:
        unregister("position", "toy_offsets")
        unregister("mixer", "toy_narrow_values")
        unregister_architecture("ToyOffsetsForCausalLM")
