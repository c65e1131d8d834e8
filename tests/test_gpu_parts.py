"""Each part of a layer alone against the plain implementation's function, and
the generality of the composition: a toy mixer with state of its own, defined
here, is registered, built into a model, loaded and stepped (whole and cut into
portions, with slot reuse) without any change to the framework's files; the run
order names a layer twice and lets a run read an earlier run's cache."""

from dataclasses import dataclass
from typing import Tuple

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def _env(dtype, page=4):
    from servelab_b200.parts import BuildEnv
    return BuildEnv(device=DEV, dtype=DT[dtype], page_size=page)


def _build(table, spec, prefix, dtype, seed=0, page=4):
    """Build one part from random tensors; returns (part, CPU float32 tensors)."""
    from servelab_b200.parts import build_part, part_class
    from servelab_b200.weights import RandomSource, WeightStore
    decls = part_class(table, spec).declare(spec, prefix)
    src = RandomSource(decls, seed, std=0.08, dtype=DT[dtype])
    part = build_part(table, spec, prefix, _env(dtype, page))
    part.load(WeightStore(src, decls, DT[dtype], DEV))
    return part, {d.name: src.read(d.name).float() for d in decls}


def _ctx(entries, groups=1):
    from servelab_b200.engine.batch import StepContext
    return StepContext.pack(entries, groups, DEV)


def _entry(tokens, start, table, want=(), slot=0):
    from servelab_b200.engine.batch import BatchEntry
    return BatchEntry(tokens=tokens, start=start, want=want, block_tables=[table], state_slot=slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from servelab_b200.config import RMSNormSpec
    from servelab_b200.parts import NORMS
    part, w = _build(NORMS, RMSNormSpec(dim=88, eps=2e-5), "n", dtype)
    resid = torch.randn(5, 88, device=DEV)
    delta = torch.randn(5, 88, device=DEV).to(DT[dtype])
    want = P.rms_norm((resid + delta.float()).cpu(), w["n.weight"], 2e-5)
    got = part.forward(None, resid, delta)
    assert got.dtype == DT[dtype] and (got.float().cpu() - want).abs().max() <= TOL[dtype] * 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter,tokens", [(172, 9), (192, 9), (192, 70), (320, 1)])
def test_feed_forward_part(dtype, inter, tokens):
    """172: gate rows then up rows.  Multiples of 64: alternating runs, with the activation
    inside the product for a few tokens in bfloat16 and in its own kernel otherwise."""
    from servelab_b200.config import GatedMLPSpec
    from servelab_b200.parts import FEED_FORWARDS
    part, w = _build(FEED_FORWARDS, GatedMLPSpec(hidden_size=72, intermediate_size=inter), "mlp", dtype)
    assert part.block == (64 if inter % 64 == 0 else 0)
    x = torch.randn(tokens, 72, device=DEV).to(DT[dtype])
    want = P.swiglu(x.float().cpu(), w["mlp.gate_proj.weight"], w["mlp.up_proj.weight"],
                    w["mlp.down_proj.weight"])
    got = part.forward(None, x)
    assert (got.float().cpu() - want).abs().max() <= TOL[dtype]


def _attention_reference(w, x, H_, Hkv, D, theta, window, rot=None):
    T = x.shape[0]
    q = P.linear(x, w["a.q_proj.weight"], w["a.q_proj.bias"]).view(T, H_, D)
    k = P.linear(x, w["a.k_proj.weight"], w["a.k_proj.bias"]).view(T, Hkv, D)
    v = P.linear(x, w["a.v_proj.weight"], w["a.v_proj.bias"]).view(T, Hkv, D)
    if theta:
        rot = rot or D
        inv, pos = P.rope_inv_freq(rot, theta), torch.arange(T)
        q = torch.cat([P.rope(q[..., :rot], pos, inv), q[..., rot:]], -1)
        k = torch.cat([P.rope(k[..., :rot], pos, inv), k[..., rot:]], -1)
    return P.linear(P.causal_attention(q, k, v, window), w["a.o_proj.weight"],
                    w.get("a.o_proj.bias"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["rotary", "window", "no_position", "partial_rotary_out_bias"])
def test_attention_mixer_alone_whole_and_in_portions(dtype, variant):
    from servelab_b200.config import AttentionSpec, NoPositionSpec, RotarySpec
    from servelab_b200.parts import MIXERS, LayerCache
    H_, Hkv, D, hid, T, ps = 6, 2, 32, 40, 29, 4
    theta, window, rot, out_bias = 10000.0, None, D, False
    if variant == "window":
        window = 5
    if variant == "no_position":
        theta = 0.0
    if variant == "partial_rotary_out_bias":
        rot, out_bias = 16, True
    pos_spec = RotarySpec(head_dim=D, rotary_dim=rot, theta=theta) if theta else NoPositionSpec()
    spec = AttentionSpec(hidden_size=hid, num_heads=H_, num_kv_heads=Hkv, head_dim=D,
                         qkv_bias=True, out_bias=out_bias, window=window, position=pos_spec)
    part, w = _build(MIXERS, spec, "a", dtype, page=ps)
    x = torch.randn(T, hid).to(DT[dtype])
    want = _attention_reference(w, x.float(), H_, Hkv, D, theta, window, rot)
    pages = [5, 0, 7, 3, 9, 1, 8, 2]
    for cuts in ([T], [3, 2, 11, 1, 1, 9, 2]):
        k = torch.zeros(10, Hkv, ps, D, device=DEV, dtype=DT[dtype])
        cache = LayerCache(group=0, k=k, v=torch.zeros_like(k), page_size=ps)
        outs, start = [], 0
        for n in cuts:
            ctx = _ctx([_entry([0] * n, start, pages[:-(-(start + n) // ps)])])
            outs.append(part.forward(ctx, x[start:start + n].to(DEV), cache, True).float().cpu())
            start += n
        got = torch.cat(outs)
        assert (got - want).abs().max() <= TOL[dtype], (variant, cuts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_alone(dtype):
    from servelab_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, RMSNormSpec,
                                      RotarySpec)
    from servelab_b200.parts import BLOCKS, LayerCache
    hid, H_, Hkv, D, I, T, ps = 48, 3, 3, 16, 100, 13, 8
    norm = RMSNormSpec(dim=hid, eps=1e-6)
    spec = BlockSpec(
        mixer=AttentionSpec(hidden_size=hid, num_heads=H_, num_kv_heads=Hkv, head_dim=D,
                            qkv_bias=True, position=RotarySpec(head_dim=D, rotary_dim=D, theta=1e4)),
        feed_forward=GatedMLPSpec(hidden_size=hid, intermediate_size=I), mixer_norm=norm, ff_norm=norm)
    part, w = _build(BLOCKS, spec, "L", dtype, page=ps)
    x = torch.randn(T, hid)
    wa = {k.replace("L.self_attn", "a"): v for k, v in w.items()}
    h1 = x + _attention_reference(wa, P.rms_norm(x, w["L.input_layernorm.weight"], 1e-6),
                                  H_, Hkv, D, 1e4, None)
    want = h1 + P.swiglu(P.rms_norm(h1, w["L.post_attention_layernorm.weight"], 1e-6),
                         w["L.mlp.gate_proj.weight"], w["L.mlp.up_proj.weight"],
                         w["L.mlp.down_proj.weight"])
    k = torch.zeros(4, Hkv, ps, D, device=DEV, dtype=DT[dtype])
    cache = LayerCache(group=0, k=k, v=torch.zeros_like(k), page_size=ps)
    resid = x.to(DEV).clone()
    ctx = _ctx([_entry([0] * T, 0, [2, 0])])
    resid, delta = part.forward(ctx, resid, None, cache, True)
    got = (resid + delta.float()).cpu()
    assert (got - want).abs().max() <= TOL[dtype] * 2


# --------------------------------------------------------------------------- #
# a toy architecture, defined entirely in this test
# --------------------------------------------------------------------------- #

def _register_toy():
    """Registers (once) a mixer with per-request state -- a running mean of its
    inputs scaled by a learned vector -- and a toy architecture that uses it."""
    from servelab_b200.cache import FixedStateRequest
    from servelab_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, LayerRun, ModelSpec,
                                      PartSpec, RMSNormSpec, RotarySpec, register_architecture)
    from servelab_b200.parts import MIXERS, Mixer, register_mixer
    from servelab_b200.weights import NORM, TensorDecl

    if "toy_running_mean" in MIXERS:
        return

    @dataclass(frozen=True)
    class RunningMeanSpec(PartSpec):
        kind: str = "toy_running_mean"
        hidden_size: int = 0

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        """y_t = gain * mean(x_0 .. x_t); the state slot holds [sum | count]."""

        @classmethod
        def declare(cls, spec, prefix):
            return [TensorDecl(prefix + ".gain", (spec.hidden_size,), NORM)]

        @classmethod
        def cache_request(cls, spec):
            return FixedStateRequest((spec.hidden_size + 1,))

        def load(self, store):
            self.gain = store.get(self.prefix + ".gain")

        # forward() launches kernels on the step's device buffers only and reads nothing of
        # the batch on the host: a decode step with this mixer can be captured in a CUDA graph
        graph_safe = True

        def forward(self, ctx, x, cache, owns_cache):
            slots, seq = ctx.state_slots.long(), ctx.seq_of_token.long()
            first = ctx.cu_q[:-1].long()                       # a request's first token of the step
            last = ctx.cu_q[1:].long() - 1
            xf = x.float()
            csum = torch.cumsum(xf, 0)                         # over the packed tokens of all requests
            before = (csum[first] - xf[first])[seq]            # ... up to the request's own first token
            state = cache.state[slots]                         # [S, hidden + 1]
            sums = state[:, :-1][seq] + csum - before
            index = torch.arange(x.shape[0], device=x.device) - first[seq] + 1
            counts = state[:, -1][seq] + index.float()
            if owns_cache:
                cache.state[slots] = torch.cat([sums[last], counts[last, None]], 1)
            return (sums / counts[:, None] * self.gain).to(x.dtype)

    class ToyConfig:
        architecture = "ToyStateForCausalLM"

        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d, architectures=[self.architecture])

        def to_model_spec(self):
            d = self.d
            hid, D = d["hidden_size"], d["head_dim"]
            norm = RMSNormSpec(dim=hid, eps=d["eps"])
            ff = GatedMLPSpec(hidden_size=hid, intermediate_size=d["intermediate_size"])
            attn = AttentionSpec(hidden_size=hid, num_heads=d["heads"], num_kv_heads=d["kv_heads"],
                                 head_dim=D, qkv_bias=True,
                                 position=RotarySpec(head_dim=D, rotary_dim=D, theta=d["theta"]))
            layers = (BlockSpec(mixer=attn, feed_forward=ff, mixer_norm=norm, ff_norm=norm),
                      BlockSpec(mixer=RunningMeanSpec(hidden_size=hid), feed_forward=ff,
                                mixer_norm=norm, ff_norm=norm))
            # layer 0, the state layer, layer 0 again with a cache of its own, then layer 0
            # reading the cache that run 0 filled
            order = (LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(0, cache_of=0))
            return ModelSpec(architecture=self.architecture, hidden_size=hid,
                             vocab_size=d["vocab_size"], layers=layers, run_order=order,
                             final_norm=norm, tie_word_embeddings=True,
                             max_position_embeddings=256)

    register_architecture(ToyConfig.architecture, ToyConfig)


TOY = {"architectures": ["ToyStateForCausalLM"], "hidden_size": 48, "head_dim": 16, "heads": 3,
       "kv_heads": 1, "intermediate_size": 56, "vocab_size": 130, "eps": 1e-6, "theta": 10000.0}


def _toy_plain(folder, ids):
    cfg, w = P.load_folder(folder)
    T, hid, D, H_, Hkv = len(ids), 48, 16, 3, 1
    x = P.embed(torch.tensor(ids), w["model.embed_tokens.weight"])
    inv, pos = P.rope_inv_freq(D, 10000.0), torch.arange(T)

    def qkv(layer, h):
        p = f"model.layers.{layer}.self_attn."
        q = P.rope(P.linear(h, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(T, H_, D), pos, inv)
        k = P.rope(P.linear(h, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(T, Hkv, D), pos, inv)
        v = P.linear(h, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(T, Hkv, D)
        return q, k, v

    def ff(layer, h):
        p = f"model.layers.{layer}."
        return P.swiglu(P.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-6),
                        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                        w[p + "mlp.down_proj.weight"])

    kv0 = None
    for run, (layer, shared) in enumerate([(0, False), (1, False), (0, False), (0, True)]):
        h = P.rms_norm(x, w[f"model.layers.{layer}.input_layernorm.weight"], 1e-6)
        if layer == 1:
            mean = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
            a = mean * w["model.layers.1.self_attn.gain"]
        else:
            q, k, v = qkv(0, h)
            if run == 0:
                kv0 = (k, v)
            if shared:
                k, v = kv0
            a = P.linear(P.causal_attention(q, k, v), w["model.layers.0.self_attn.o_proj.weight"])
        x = x + a
        x = x + ff(layer, x)
    return P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-6),
                    w["model.embed_tokens.weight"]).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype, tmp_path):
    _register_toy()
    from servelab_b200.config import config_from_dict
    from servelab_b200.replay import TraceSession
    from servelab_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "toy"), config_from_dict(TOY), seed=5)
    reqs = {f"t{i}": H.random_ids(n, 130, 50 + i) for i, n in enumerate([41, 60, 35, 52])}
    ref = {rid: _toy_plain(folder, ids) for rid, ids in reqs.items()}
    for steps in (H.trace_whole(reqs), H.trace_portions(reqs),
                  H.trace_mixed(reqs, seed=2, max_live=2)):
        sess = TraceSession(folder, dtype, H.peak_tokens(steps), page_size=8, max_live=2)
        storage = sess.runner.storage
        assert len(storage.groups) == 1 and len(storage.groups[0].layers) == 2   # runs 0 and 2
        assert storage.state_layers == [1]
        got = H.collect(steps, H.run_session(sess, steps), 130)
        for rid, ids in reqs.items():
            for pos in range(len(ids)):
                err = float(np.abs(got[rid][pos] - ref[rid][pos]).max())
                assert err <= TOL[dtype] * 2, (rid, pos, err)
        sess.cache.check_invariants()
        assert sess.cache.slots.num_free() == 2


def test_toy_mixer_with_state_decodes_through_replayed_graphs(tmp_path):
    """The stateful mixer declares itself graph-safe like every other part: steps of single
    tokens replay a captured graph (the state is indexed by the step's slot ids on the
    device), and the logits are those of the eager steps.  Two requests, so that the second
    takes a slot the first has used."""
    _register_toy()
    from servelab_b200.config import config_from_dict
    from servelab_b200.replay import TraceSession
    from servelab_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "toy"), config_from_dict(TOY), seed=5)
    reqs = {f"t{i}": H.random_ids(n, 130, 70 + i) for i, n in enumerate([44, 39])}
    ref = {rid: _toy_plain(folder, ids) for rid, ids in reqs.items()}
    steps = H.trace_bulk_tail(reqs, tail=20)
    for dtype in ("float32", "bfloat16"):
        sess = TraceSession(folder, dtype, H.peak_tokens(steps), page_size=8, max_live=1, cuda_graphs=True)
        assert sess.runner.storage.state_layers == [1] and sess.runner._graph_safe
        got = H.collect(steps, H.run_session(sess, steps), 130)
        assert sess.runner.graph_replays == 40
        for rid, ids in reqs.items():
            for pos in range(len(ids)):
                err = float(np.abs(got[rid][pos] - ref[rid][pos]).max())
                assert err <= TOL[dtype] * 2, (dtype, rid, pos, err)


# --------------------------------------------------------------------------- #
# another position encoding, defined in this test: learned absolute positions
# --------------------------------------------------------------------------- #

def _register_learned_positions():
    from servelab_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, LayerRun, ModelSpec,
                                      NoPositionSpec, PartSpec, RMSNormSpec, register_architecture)
    from servelab_b200.parts import POSITIONS, PositionEncoding, register_position
    from servelab_b200.weights import MATRIX, TensorDecl

    if "toy_learned_absolute" in POSITIONS:
        return

    @dataclass(frozen=True)
    class LearnedSpec(PartSpec):
        kind: str = "toy_learned_absolute"
        max_positions: int = 0
        hidden_size: int = 0

    @register_position("toy_learned_absolute")
    class LearnedAbsolute(PositionEncoding):
        """resid[t] += table[position[t]]: acts on the embedded tokens, not in the mixer."""

        @classmethod
        def declare(cls, spec, prefix):
            return [TensorDecl(prefix + ".weight", (spec.max_positions, spec.hidden_size), MATRIX)]

        def load(self, store):
            self.table = store.get(self.prefix + ".weight")

        def apply_to_embedding(self, ctx, resid):
            resid += self.table[ctx.positions.long()].float()

    class ToyAbsConfig:
        architecture = "ToyAbsoluteForCausalLM"

        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d, architectures=[self.architecture])

        def to_model_spec(self):
            d = self.d
            hid = d["hidden_size"]
            norm = RMSNormSpec(dim=hid, eps=1e-5)
            attn = AttentionSpec(hidden_size=hid, num_heads=2, num_kv_heads=2, head_dim=hid // 2,
                                 qkv_bias=False, position=NoPositionSpec())
            block = BlockSpec(mixer=attn, feed_forward=GatedMLPSpec(hidden_size=hid, intermediate_size=72),
                              mixer_norm=norm, ff_norm=norm)
            return ModelSpec(architecture=self.architecture, hidden_size=hid, vocab_size=d["vocab_size"],
                             layers=(block, block), run_order=(LayerRun(0), LayerRun(1)),
                             final_norm=norm, tie_word_embeddings=False, max_position_embeddings=128,
                             embedding_position=LearnedSpec(max_positions=128, hidden_size=hid))

    register_architecture(ToyAbsConfig.architecture, ToyAbsConfig)


def _toy_abs_plain(folder, ids):
    _, w = P.load_folder(folder)
    T, hid = len(ids), 32
    x = P.embed(torch.tensor(ids), w["model.embed_tokens.weight"]) + w["model.embed_positions.weight"][:T]
    for layer in range(2):
        p = f"model.layers.{layer}."
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
        q = P.linear(h, w[p + "self_attn.q_proj.weight"]).view(T, 2, 16)
        k = P.linear(h, w[p + "self_attn.k_proj.weight"]).view(T, 2, 16)
        v = P.linear(h, w[p + "self_attn.v_proj.weight"]).view(T, 2, 16)
        x = x + P.linear(P.causal_attention(q, k, v), w[p + "self_attn.o_proj.weight"])
        x = x + P.swiglu(P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5),
                         w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                         w[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"]).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_position_encoding_defined_in_the_test(dtype, tmp_path):
    _register_learned_positions()
    from servelab_b200.config import config_from_dict
    from servelab_b200.replay import TraceSession
    from servelab_b200.weights import write_random_model
    cfg = {"architectures": ["ToyAbsoluteForCausalLM"], "hidden_size": 32, "vocab_size": 90}
    folder = write_random_model(str(tmp_path / "abs"), config_from_dict(cfg), seed=9)
    reqs = {f"p{i}": H.random_ids(n, 90, 20 + i) for i, n in enumerate([37, 50])}
    ref = {rid: _toy_abs_plain(folder, ids) for rid, ids in reqs.items()}
    for steps in (H.trace_whole(reqs), H.trace_mixed(reqs, seed=4, max_live=2, tail=10)):
        sess = TraceSession(folder, dtype, H.peak_tokens(steps), page_size=8, max_live=2)
        got = H.collect(steps, H.run_session(sess, steps), 90)
        for rid, ids in reqs.items():
            for pos in range(len(ids)):
                assert float(np.abs(got[rid][pos] - ref[rid][pos]).max()) <= TOL[dtype] * 2, (rid, pos)


# --------------------------------------------------------------------------- #
# a feed-forward with routing, defined in this test (top-1 of three experts)
# --------------------------------------------------------------------------- #

def _register_routed_ff():
    from servelab_b200.config import (AttentionSpec, BlockSpec, LayerRun, ModelSpec, PartSpec,
                                      RMSNormSpec, RotarySpec, register_architecture)
    from servelab_b200.ops.linear import linear
    from servelab_b200.parts import FEED_FORWARDS, FeedForward, register_feed_forward
    from servelab_b200.weights import MATRIX, TensorDecl

    if "toy_top1_experts" in FEED_FORWARDS:
        return

    @dataclass(frozen=True)
    class RoutedSpec(PartSpec):
        kind: str = "toy_top1_experts"
        hidden_size: int = 0
        intermediate_size: int = 0
        num_experts: int = 0

    @register_feed_forward("toy_top1_experts")
    class Top1Experts(FeedForward):
        """Router logits in float32; each token goes through the one expert with the
        largest logit (relu MLP), weighted by the softmax probability of that expert."""

        @classmethod
        def declare(cls, spec, prefix):
            out = [TensorDecl(prefix + ".router.weight", (spec.num_experts, spec.hidden_size), MATRIX)]
            for e in range(spec.num_experts):
                out += [TensorDecl(f"{prefix}.experts.{e}.up.weight",
                                   (spec.intermediate_size, spec.hidden_size), MATRIX),
                        TensorDecl(f"{prefix}.experts.{e}.down.weight",
                                   (spec.hidden_size, spec.intermediate_size), MATRIX)]
            return out

        def load(self, store):
            self.router = store.get(self.prefix + ".router.weight").float()
            self.up = [store.get(f"{self.prefix}.experts.{e}.up.weight") for e in range(self.spec.num_experts)]
            self.down = [store.get(f"{self.prefix}.experts.{e}.down.weight") for e in range(self.spec.num_experts)]

        def forward(self, ctx, x):
            probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
            choice = probs.argmax(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.spec.num_experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                h = torch.relu(linear(x[rows].contiguous(), self.up[e]))
                y = linear(h, self.down[e]).float() * probs[rows, e][:, None]
                out[rows] = y.to(x.dtype)
            return out

    class ToyMoEConfig:
        architecture = "ToyRoutedForCausalLM"

        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d, architectures=[self.architecture])

        def to_model_spec(self):
            hid = self.d["hidden_size"]
            norm = RMSNormSpec(dim=hid, eps=1e-6)
            attn = AttentionSpec(hidden_size=hid, num_heads=2, num_kv_heads=1, head_dim=16,
                                 qkv_bias=True, position=RotarySpec(head_dim=16, rotary_dim=16, theta=1e4))
            ff = RoutedSpec(hidden_size=hid, intermediate_size=48, num_experts=3)
            block = BlockSpec(mixer=attn, feed_forward=ff, mixer_norm=norm, ff_norm=norm)
            return ModelSpec(architecture=self.architecture, hidden_size=hid,
                             vocab_size=self.d["vocab_size"], layers=(block, block),
                             run_order=(LayerRun(0), LayerRun(1)), final_norm=norm,
                             tie_word_embeddings=True, max_position_embeddings=128)

    register_architecture(ToyMoEConfig.architecture, ToyMoEConfig)


def _toy_routed_plain(folder, ids):
    _, w = P.load_folder(folder)
    T = len(ids)
    x = P.embed(torch.tensor(ids), w["model.embed_tokens.weight"])
    inv, pos = P.rope_inv_freq(16, 1e4), torch.arange(T)
    for layer in range(2):
        p = f"model.layers.{layer}."
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
        q = P.rope(P.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, 2, 16), pos, inv)
        k = P.rope(P.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(T, 1, 16), pos, inv)
        v = P.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(T, 1, 16)
        x = x + P.linear(P.causal_attention(q, k, v), w[p + "self_attn.o_proj.weight"])
        h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-6)
        probs = torch.softmax(P.linear(h, w[p + "mlp.router.weight"]), dim=-1)
        choice = probs.argmax(-1)
        y = torch.zeros_like(h)
        for t in range(T):
            e = int(choice[t])
            hid = torch.relu(P.linear(h[t:t + 1], w[f"{p}mlp.experts.{e}.up.weight"]))
            y[t] = P.linear(hid, w[f"{p}mlp.experts.{e}.down.weight"])[0] * probs[t, e]
        x = x + y
    return P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-6), w["model.embed_tokens.weight"]).numpy()


def test_feed_forward_with_routing_defined_in_the_test(tmp_path):
    """float32 only: with bfloat16 a near-tie of router logits may pick another expert."""
    _register_routed_ff()
    from servelab_b200.config import config_from_dict
    from servelab_b200.replay import TraceSession
    from servelab_b200.weights import write_random_model
    cfg = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 32, "vocab_size": 70}
    folder = write_random_model(str(tmp_path / "moe"), config_from_dict(cfg), seed=3, std=0.2)
    reqs = {f"m{i}": H.random_ids(n, 70, 40 + i) for i, n in enumerate([33, 41])}
    ref = {rid: _toy_routed_plain(folder, ids) for rid, ids in reqs.items()}
    for steps in (H.trace_whole(reqs), H.trace_mixed(reqs, seed=6, max_live=2, tail=10)):
        sess = TraceSession(folder, "float32", H.peak_tokens(steps), page_size=8, max_live=2)
        got = H.collect(steps, H.run_session(sess, steps), 70)
        for rid, ids in reqs.items():
            for pos in range(len(ids)):
                assert float(np.abs(got[rid][pos] - ref[rid][pos]).max()) <= 5e-5, (rid, pos)


# --------------------------------------------------------------------------- #
# K-split partial sums handed to the consuming kernels (an optional path)
# --------------------------------------------------------------------------- #

def test_split_sums_consumed_by_norm_and_rope_kernels(tmp_path):
    """The ways a decode step sums the K splits of its narrow products: a reduction kernel,
    float32 partial sums that the norm / rotary kernels add (``defer_split_sums``), and
    thread-block clusters that add them through shared memory, with and without the
    rotation and cache write in the q|k|v product's epilogue, and with and without the
    residual add and the norm in the epilogue of the o and down products.  Logits must agree with the
    plain implementation and with one another whichever runs."""
    from servelab_b200.ops import kernels as kernels_module
    from servelab_b200.ops import linear as linear_ops
    from servelab_b200.replay import TraceSession
    cfg = dict(H.TINY_B, hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
               intermediate_size=1024)
    folder = H.make_model(str(tmp_path / "m"), cfg, 4)
    reqs = {"a": H.random_ids(40, 512, 1), "b": H.random_ids(37, 512, 2)}
    steps = H.trace_bulk_tail(reqs, tail=16)
    outs = {}
    saved = (dict(linear_ops.defer_split_sums), linear_ops.cluster_sums, linear_ops.fuse_qkv_rope,
             linear_ops.fuse_resid_norm)
    modes = {"reduce": (False, False, False, False), "parts": (True, False, False, False),
             "cluster": (True, True, False, False), "cluster+rope": (True, True, True, False),
             "cluster+norm": (True, True, False, True), "cluster+rope+norm": (True, True, True, True)}
    for name, (defer, cluster, rope, norm) in modes.items():
        linear_ops.defer_split_sums.update(rope=defer, norm=defer)
        linear_ops.cluster_sums, linear_ops.fuse_qkv_rope, linear_ops.fuse_resid_norm = cluster, rope, norm
        try:
            before = kernels_module.launch_count
            sess = TraceSession(folder, "bfloat16", H.peak_tokens(steps), page_size=8, max_live=2)
            outs[name] = H.collect(steps, H.run_session(sess, steps), 512)
            outs[name + " launches"] = kernels_module.launch_count - before
        finally:
            linear_ops.defer_split_sums.update(saved[0])
            linear_ops.cluster_sums, linear_ops.fuse_qkv_rope, linear_ops.fuse_resid_norm = saved[1:]
    assert kernels_module.gemm_tc_status(True) == 0
    # fewer kernels run, form by form
    assert outs["reduce launches"] > outs["parts launches"] >= outs["cluster launches"] \
        > outs["cluster+rope launches"] > outs["cluster+rope+norm launches"]
    assert outs["cluster launches"] > outs["cluster+norm launches"]
    ref = {rid: H.plain_logits(folder, ids) for rid, ids in reqs.items()}
    for name in modes:
        for rid, ids in reqs.items():
            for pos in range(len(ids)):
                assert float(np.abs(outs[name][rid][pos] - ref[rid][pos]).max()) <= 3e-2, name
                assert float(np.abs(outs[name][rid][pos] - outs["reduce"][rid][pos]).max()) <= 2e-2, name


# --------------------------------------------------------------------------- #
# a position encoding that acts on q and k and is no rotation, defined in this test
# --------------------------------------------------------------------------- #

def _register_qk_positions():
    from servelab_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, LayerRun, ModelSpec,
                                      PartSpec, RMSNormSpec, register_architecture)
    from servelab_b200.parts import POSITIONS, PositionEncoding, register_position

    if "toy_position_gain" in POSITIONS:
        return

    @dataclass(frozen=True)
    class GainSpec(PartSpec):
        kind: str = "toy_position_gain"
        head_dim: int = 0

    @register_position("toy_position_gain")
    class PositionGain(PositionEncoding):
        """q and k are multiplied, element by element, by 1 + 0.5 sin(position * f_d): an
        encoding inside the scores that is no rotation, so it cannot ride in the mixer's
        rotary kernel and uses the ``apply_to_qk`` seam instead."""
        transforms_qk = True
        graph_safe = True

        def __init__(self, spec, prefix, env):
            super().__init__(spec, prefix, env)
            self.freq = (0.3 + 0.05 * torch.arange(spec.head_dim, dtype=torch.float32)).to(env.device)

        def apply_to_qk(self, ctx, q, k):
            gain = 1.0 + 0.5 * torch.sin(ctx.positions.float()[:, None] * self.freq[None, :])   # [T, D]
            q.mul_(gain[:, None, :].to(q.dtype))
            k.mul_(gain[:, None, :].to(k.dtype))

    class ToyGainConfig:
        architecture = "ToyGainForCausalLM"

        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d, architectures=[self.architecture])

        def to_model_spec(self):
            hid = self.d["hidden_size"]
            norm = RMSNormSpec(dim=hid, eps=1e-5)
            attn = AttentionSpec(hidden_size=hid, num_heads=4, num_kv_heads=2, head_dim=hid // 4,
                                 qkv_bias=True, position=GainSpec(head_dim=hid // 4))
            block = BlockSpec(mixer=attn, feed_forward=GatedMLPSpec(hidden_size=hid, intermediate_size=80),
                              mixer_norm=norm, ff_norm=norm)
            return ModelSpec(architecture=self.architecture, hidden_size=hid, vocab_size=self.d["vocab_size"],
                             layers=(block, block), run_order=(LayerRun(0), LayerRun(1)), final_norm=norm,
                             tie_word_embeddings=True, max_position_embeddings=128)

    register_architecture(ToyGainConfig.architecture, ToyGainConfig)


def _toy_gain_plain(folder, ids):
    _, w = P.load_folder(folder)
    T, hid, Hq, Hkv, D = len(ids), 64, 4, 2, 16
    gain = 1.0 + 0.5 * torch.sin(torch.arange(T).float()[:, None] * (0.3 + 0.05 * torch.arange(D).float())[None, :])
    x = P.embed(torch.tensor(ids), w["model.embed_tokens.weight"])
    for layer in range(2):
        p = f"model.layers.{layer}."
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
        q = P.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, Hq, D)
        k = P.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(T, Hkv, D)
        v = P.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(T, Hkv, D)
        a = P.causal_attention(q * gain[:, None, :], k * gain[:, None, :], v)
        x = x + P.linear(a, w[p + "self_attn.o_proj.weight"])
        x = x + P.swiglu(P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5),
                         w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                         w[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-5), w["model.embed_tokens.weight"]).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_position_encoding_inside_the_scores_that_is_no_rotation(dtype, tmp_path):
    _register_qk_positions()
    from servelab_b200.config import config_from_dict
    from servelab_b200.replay import TraceSession
    from servelab_b200.weights import write_random_model
    cfg = {"architectures": ["ToyGainForCausalLM"], "hidden_size": 64, "vocab_size": 110}
    folder = write_random_model(str(tmp_path / "gain"), config_from_dict(cfg), seed=21,
                                std_of={"q_proj.weight": 0.15, "k_proj.weight": 0.15})
    reqs = {f"g{i}": H.random_ids(n, 110, 30 + i) for i, n in enumerate([45, 61])}
    ref = {rid: _toy_gain_plain(folder, ids) for rid, ids in reqs.items()}
    for steps in (H.trace_whole(reqs), H.trace_mixed(reqs, seed=6, max_live=2, tail=12)):
        sess = TraceSession(folder, dtype, H.peak_tokens(steps), page_size=8, max_live=2,
                            cuda_graphs=True)
        got = H.collect(steps, H.run_session(sess, steps), 110)
        for rid, ids in reqs.items():
            for pos in range(len(ids)):
                err = float(np.abs(got[rid][pos] - ref[rid][pos]).max())
                assert err <= (1e-4 if dtype == "float32" else 5e-2), (rid, pos, err)


# --------------------------------------------------------------------------- #
# an architecture with the same parts under other tensor names, an embedding scale
# and transformed logits: a config class alone, nothing else
# --------------------------------------------------------------------------- #

_RENAMED_LAYER = {"input_layernorm": "ln_1", "self_attn": "attn", "post_attention_layernorm": "ln_2",
                  "mlp": "ffn", "q_proj": "wq", "k_proj": "wk", "v_proj": "wv", "o_proj": "wo",
                  "gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}
_EMBED_SCALE, _LOGIT_SCALE, _SOFTCAP = 6.0, 0.5, 0.8


def _register_renamed():
    from servelab_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, LayerRun, ModelSpec,
                                      RMSNormSpec, RotarySpec, register_architecture,
                                      registered_architectures)
    if "ToyRenamedForCausalLM" in registered_architectures():
        return

    class ToyRenamedConfig:
        architecture = "ToyRenamedForCausalLM"

        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d, architectures=[self.architecture])

        def to_model_spec(self):
            d, n = self.d, _RENAMED_LAYER
            hid, D = d["hidden_size"], d["head_dim"]
            norm = RMSNormSpec(dim=hid, eps=d["eps"])
            attn = AttentionSpec(hidden_size=hid, num_heads=d["heads"], num_kv_heads=d["kv_heads"], head_dim=D,
                                 qkv_bias=True, position=RotarySpec(head_dim=D, rotary_dim=D, theta=d["theta"]),
                                 q_name=n["q_proj"], k_name=n["k_proj"], v_name=n["v_proj"], o_name=n["o_proj"])
            ff = GatedMLPSpec(hidden_size=hid, intermediate_size=d["intermediate_size"],
                              gate_name=n["gate_proj"], up_name=n["up_proj"], down_name=n["down_proj"])
            block = BlockSpec(mixer=attn, feed_forward=ff, mixer_norm=norm, ff_norm=norm,
                              mixer_norm_name=n["input_layernorm"], mixer_name=n["self_attn"],
                              ff_norm_name=n["post_attention_layernorm"], feed_forward_name=n["mlp"])
            L = d["layers"]
            return ModelSpec(architecture=self.architecture, hidden_size=hid, vocab_size=d["vocab_size"],
                             layers=(block,) * L, run_order=tuple(LayerRun(i) for i in range(L)),
                             final_norm=norm, tie_word_embeddings=False, max_position_embeddings=256,
                             embed_name="transformer.wte.weight", lm_head_name="output.weight",
                             final_norm_prefix="transformer.ln_f", layer_prefix="transformer.h.{}",
                             embedding_scale=_EMBED_SCALE, logit_scale=_LOGIT_SCALE, logit_softcap=_SOFTCAP)

    register_architecture(ToyRenamedConfig.architecture, ToyRenamedConfig)


def _renamed_plain(folder, cfg, ids):
    """The plain Qwen2 implementation on the same tensors under its own names, with the scaled
    embedding table; then the logit transform."""
    _, w = P.load_folder(folder)
    back = {v: k for k, v in _RENAMED_LAYER.items()}
    renamed = {}
    for name, t in w.items():
        parts = name.split(".")
        if parts[0] == "transformer" and parts[1] == "h":
            renamed[".".join(["model", "layers", parts[2]] + [back.get(p, p) for p in parts[3:]])] = t
    renamed["model.embed_tokens.weight"] = w["transformer.wte.weight"] * _EMBED_SCALE
    renamed["model.norm.weight"] = w["transformer.ln_f.weight"]
    renamed["lm_head.weight"] = w["output.weight"]
    qcfg = {"num_hidden_layers": cfg["layers"], "hidden_size": cfg["hidden_size"],
            "num_attention_heads": cfg["heads"], "num_key_value_heads": cfg["kv_heads"],
            "head_dim": cfg["head_dim"], "rms_norm_eps": cfg["eps"], "rope_theta": cfg["theta"],
            "tie_word_embeddings": False}
    logits = P.forward_logits(qcfg, renamed, ids) * _LOGIT_SCALE
    return (_SOFTCAP * torch.tanh(logits / _SOFTCAP)).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_architecture_with_other_tensor_names_and_scales_is_a_config_class_alone(dtype, tmp_path):
    _register_renamed()
    from servelab_b200.config import config_from_dict
    from servelab_b200.models import declare_tensors
    from servelab_b200.replay import TraceSession
    from servelab_b200.weights import write_random_model
    cfg = {"architectures": ["ToyRenamedForCausalLM"], "hidden_size": 64, "head_dim": 16, "heads": 4,
           "kv_heads": 2, "intermediate_size": 128, "vocab_size": 150, "layers": 2, "eps": 1e-5,
           "theta": 10000.0}
    config = config_from_dict(cfg)
    names = {d.name for d in declare_tensors(config.to_model_spec())}
    assert "transformer.h.1.attn.wk.bias" in names and "transformer.h.0.ffn.w3.weight" in names
    assert "transformer.wte.weight" in names and "output.weight" in names
    assert not any("self_attn" in n or "mlp" in n or n.startswith("model.") for n in names)
    folder = write_random_model(str(tmp_path / "renamed"), config, seed=31, std_of={"output.weight": 0.3})
    reqs = {f"n{i}": H.random_ids(n, 150, 40 + i) for i, n in enumerate([52, 47])}
    ref = {rid: _renamed_plain(folder, cfg, ids) for rid, ids in reqs.items()}
    assert max(float(np.abs(r).max()) for r in ref.values()) > 0.5 * _SOFTCAP, "the cap must bite"
    for steps in (H.trace_whole(reqs), H.trace_bulk_tail(reqs, tail=12)):
        sess = TraceSession(folder, dtype, H.peak_tokens(steps), page_size=16, max_live=2, cuda_graphs=True)
        got = H.collect(steps, H.run_session(sess, steps), 150)
        for rid, ids in reqs.items():
            for pos in range(len(ids)):
                err = float(np.abs(got[rid][pos] - ref[rid][pos]).max())
                assert err <= (2e-5 if dtype == "float32" else 3e-2), (rid, pos, err)
