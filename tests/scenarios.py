"""Scenarios that run the engine against the plain implementation.  Each takes the device
and dtype: the host-side tests run them on the CPU with the stand-in kernels
(tests/fake_ops.py), the GPU tests run them on cuda:0 with the real ones."""
from __future__ import annotations

import copy
import os
from dataclasses import dataclass, replace
from typing import List

import torch

import helpers
from plain import qwen2_plain as plain


def runner_for(folder, device, dtype, num_pages, max_requests=4, max_seq_len=None, page_size=16):
    from vt_transformer_b200.engine.runner import ModelRunner
    return ModelRunner.from_folder(folder, dtype=dtype, device=device, page_size=page_size, num_pages=num_pages,
                                   max_requests=max_requests, max_seq_len=max_seq_len)


# ----------------------------------------------------------------------------- the four ways of cutting


def replay_family(folder, name, family, device, dtype):
    prompts = helpers.prompts_for(name)
    trace = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda p: helpers.trace_mixed(p, max_live=4, seed=3)}[family](prompts)
    # so few pages that they are used again: what the live requests need at most, no more
    pages = helpers.tokens_needed(trace, round_to=16) // 16
    runner = runner_for(folder, device, dtype, num_pages=pages)
    got = helpers.run_trace_inproc(runner, trace)
    worst = helpers.compare_trace(folder, prompts, trace, got, helpers.tol(dtype, name))
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.groups]
    return worst


# ----------------------------------------------------------------------------- run order as data


def register_order_architecture(order_name: str, order):
    """An architecture that is Qwen2's parts in another run order (a test's own, never a model of
    anyone's): ``order`` is a tuple of RunSpec."""
    from vt_transformer_b200.config import Qwen2Config, register_architecture
    from vt_transformer_b200.models.qwen2 import qwen2_model_spec

    def spec(cfg):
        return replace(qwen2_model_spec(cfg), order=tuple(order))

    register_architecture(order_name, Qwen2Config, spec, replace=True)


def run_order_case(tmp, device, dtype):
    """Layer 1 runs twice (each run with a cache slot of its own) and a last run of layer 0
    reads the keys and values that the first run stored."""
    from vt_transformer_b200.config import config_from_dict, unregister_architecture
    from vt_transformer_b200.parts import RunSpec
    from vt_transformer_b200.weights import write_random_model
    order = (RunSpec(0, 0), RunSpec(1, 1), RunSpec(1, 2), RunSpec(0, 0, writes=False))
    register_order_architecture("OrderTestLM", order)
    try:
        d = copy.deepcopy(helpers.CONFIGS["A"])
        d["architectures"] = ["OrderTestLM"]
        folder = write_random_model(config_from_dict(d), os.path.join(tmp, "order"), seed=4, sigma=0.08)
        cfg, w = plain.read_config(folder), plain.read_weights(folder)
        ids = helpers.prompts_for("A")[3]
        ref = plain.forward(cfg, w, ids, order=[0, 1, 1, (0, 0)])
        runner = runner_for(folder, device, dtype, num_pages=6, max_requests=2)
        assert sorted(runner.model.cache_slots()) == [0, 1, 2]
        row = runner.admit()
        got, a = [], 0
        for k in (23, 1, 1, 30, 15):
            got.append(runner.step([helpers_entry(row, ids[a:a + k])]).float().cpu())
            a += k
        runner.check_status()
        err = float((torch.cat(got).double() - ref).abs().max())
        assert err <= helpers.tol(dtype, ref=ref), err
        plain_default = plain.forward(cfg, w, ids)
        assert float((ref - plain_default).abs().max()) > 5 * helpers.tol(dtype, ref=ref)    # the order matters
        return err
    finally:
        unregister_architecture("OrderTestLM")


def helpers_entry(row, tokens):
    from vt_transformer_b200.engine.batch import StepEntry
    return StepEntry(row, list(tokens), list(range(len(tokens))))


# ----------------------------------------------------------------------------- a toy mixer with state


def define_toy_parts():
    """A mixer that keeps state of fixed size for each request: the running mean of its inputs
    over the request's tokens, times a matrix.  Defined here, in the tests, and registered
    through the package's public registry; no file of the package knows it."""
    from vt_transformer_b200.parts import Mixer, MixerSpec, ParamSpec, StateSpec, register_part

    @dataclass(frozen=True)
    class RunningMeanSpec(MixerSpec):
        hidden: int = 0
        kind: str = "toy_running_mean"

    class RunningMean(Mixer):
        def cache_spec(self):
            return StateSpec((self.spec.hidden + 1,), torch.float32)     # sum of inputs, and their count

        def param_specs(self):
            return {self.prefix + "proj.weight": ParamSpec((self.spec.hidden, self.spec.hidden))}

        def load(self, get):
            self.w = self.rt.param(get(self.prefix + "proj.weight"))

        def forward(self, h, ctx, cache):
            out = torch.empty_like(h)
            H = self.spec.hidden
            for s in ctx.seqs:                                   # portions of a request come in order
                x = h[s.offset:s.offset + s.length].float()
                st = cache.state[s.row]
                total = st[:H] + torch.cumsum(x, dim=0)
                count = st[H] + torch.arange(1, s.length + 1, device=h.device, dtype=torch.float32)
                out[s.offset:s.offset + s.length] = ((total / count[:, None]) @ self.w.float().t()).to(h.dtype)
                st[:H] = total[-1]
                st[H] = count[-1]
            return out

    register_part("mixer", "toy_running_mean", RunningMean, replace=True)
    return RunningMeanSpec


def toy_state_case(tmp, device, dtype):
    """A model of three layers whose middle mixer is the toy: registered, built from a folder,
    stepped in portions beside another request, with its rows used again."""
    from vt_transformer_b200.config import Qwen2Config, config_from_dict, register_architecture, unregister_architecture
    from vt_transformer_b200.models.qwen2 import qwen2_model_spec
    from vt_transformer_b200.parts import unregister_part
    from vt_transformer_b200.weights import write_random_model
    Spec = define_toy_parts()

    def spec(cfg):
        base = qwen2_model_spec(cfg)
        blocks = list(base.blocks)
        blocks[1] = replace(blocks[1], mixer=Spec(hidden=cfg.hidden_size), mixer_prefix="mixer.")
        return replace(base, blocks=tuple(blocks))

    register_architecture("ToyStateLM", Qwen2Config, spec, replace=True)
    try:
        d = copy.deepcopy(helpers.CONFIGS["B"])
        d["architectures"] = ["ToyStateLM"]
        folder = write_random_model(config_from_dict(d), os.path.join(tmp, "toy"), seed=9, sigma=0.05)
        cfg, w = plain.read_config(folder), plain.read_weights(folder)
        assert "model.layers.1.mixer.proj.weight" in w and "model.layers.1.self_attn.q_proj.weight" not in w

        def reference(ids):
            cos, sin = plain.rotation_table(cfg.max_pos, cfg.head_dim, cfg.theta)
            x = plain.embed(w["model.embed_tokens.weight"], ids)
            x = plain.layer(cfg, w, 0, x, cos, sin)
            h = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], cfg.eps)
            mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1, dtype=h.dtype)[:, None]
            x = x + mean @ w["model.layers.1.mixer.proj.weight"].t()
            h = plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], cfg.eps)
            x = x + plain.swiglu(h, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"],
                                 w["model.layers.1.mlp.down_proj.weight"])
            x = plain.layer(cfg, w, 2, x, cos, sin)
            x = plain.rms_norm(x, w["model.norm.weight"], cfg.eps)
            return plain.linear(x, w["lm_head.weight"])

        runner = runner_for(folder, device, dtype, num_pages=8, max_requests=2)
        slots = runner.model.cache_slots()
        assert type(slots[1]).__name__ == "StateSpec" and type(slots[0]).__name__ == "KVCacheSpec"
        prompts = helpers.prompts_for("B")
        worst = 0.0
        for first, second in ((prompts[3], prompts[2]), (prompts[2], prompts[1])):   # the second pair uses the rows again
            rows = [runner.admit(), runner.admit()]
            got = [[], []]
            done = [0, 0]
            sizes = [[9, 2, 30, 1, 1, 27], [5, 1, 1, 13, 11]]
            for step in range(6):
                entries = []
                for i, ids in enumerate((first, second)):
                    if step < len(sizes[i]) and done[i] < len(ids):
                        k = min(sizes[i][step], len(ids) - done[i])
                        entries.append((i, helpers_entry(rows[i], ids[done[i]:done[i] + k])))
                        done[i] += k
                logits = runner.step([e for _, e in entries]).float().cpu()
                at = 0
                for i, e in entries:
                    got[i].append(logits[at:at + len(e.tokens)])
                    at += len(e.tokens)
            runner.check_status()
            for i, ids in enumerate((first, second)):
                assert done[i] == len(ids)
                ref = reference(ids)
                err = float((torch.cat(got[i]).double() - ref).abs().max())
                assert err <= helpers.tol(dtype, ref=ref), (i, err)
                worst = max(worst, err)
            for r in rows:
                runner.release(r)
        return worst
    finally:
        unregister_architecture("ToyStateLM")
        unregister_part("mixer", "toy_running_mean")


def define_toy_routed_parts():
    """A feed-forward with routing (a router picks one of the experts for every token and weighs it by the
    router's softmax) and another position encoding (rotation by angles that grow linearly with the index of the
    pair, not geometrically).  Defined here, in the tests, registered through the public registry."""
    from vt_transformer_b200.parts import FeedForward, FeedForwardSpec, ParamSpec, PositionEncoding, PositionSpec, register_part

    @dataclass(frozen=True)
    class RoutedSpec(FeedForwardSpec):
        hidden: int = 0
        inter: int = 0
        experts: int = 2
        kind: str = "toy_routed"

    class Routed(FeedForward):
        def param_specs(self):
            s, out = self.spec, {self.prefix + "router.weight": ParamSpec((self.spec.experts, self.spec.hidden))}
            for e in range(s.experts):
                out[self.prefix + f"experts.{e}.w1.weight"] = ParamSpec((s.inter, s.hidden))
                out[self.prefix + f"experts.{e}.w2.weight"] = ParamSpec((s.hidden, s.inter))
            return out

        def load(self, get):
            s = self.spec
            self.router = self.rt.param(get(self.prefix + "router.weight")).float()          # router logits in 32-bit
            self.w1 = [self.rt.param(get(self.prefix + f"experts.{e}.w1.weight")) for e in range(s.experts)]
            self.w2 = [self.rt.param(get(self.prefix + f"experts.{e}.w2.weight")) for e in range(s.experts)]

        def forward(self, h, ctx):
            ops = self.rt.ops
            prob = torch.softmax(h.float() @ self.router.t(), dim=-1)
            weight, choice = prob.max(dim=-1)
            out = torch.zeros_like(h)
            for e in range(self.spec.experts):
                idx = torch.nonzero(choice == e).flatten()
                if idx.numel() == 0:
                    continue
                x = h[idx].contiguous()
                mid = torch.empty((x.shape[0], self.spec.inter), dtype=h.dtype, device=h.device)
                ops.linear(x, self.w1[e], None, mid)
                mid = (mid.float() * torch.sigmoid(mid.float())).to(h.dtype)
                y = torch.empty((x.shape[0], self.spec.hidden), dtype=h.dtype, device=h.device)
                ops.linear(mid, self.w2[e], None, y)
                out[idx] = (y.float() * weight[idx, None]).to(h.dtype)
            return out

    @dataclass(frozen=True)
    class LinearAnglesSpec(PositionSpec):
        step: float = 0.0
        kind: str = "toy_linear_angles"

    class LinearAngles(PositionEncoding):
        def load(self, get):
            s = self.spec
            angle = torch.arange(s.max_positions, dtype=torch.float64)[:, None] * (
                s.step * torch.arange(1, s.dim // 2 + 1, dtype=torch.float64))[None, :]
            self.table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).float().contiguous().to(self.rt.device)

    register_part("feed_forward", "toy_routed", Routed, replace=True)
    register_part("position", "toy_linear_angles", LinearAngles, replace=True)
    return RoutedSpec, LinearAnglesSpec


def toy_routed_case(tmp, device, dtype):
    """A model whose first layer has the routed feed-forward and whose second layer's attention has the other
    position encoding: registered from here, built from a folder, stepped whole, in portions and token by token."""
    from vt_transformer_b200.config import Qwen2Config, config_from_dict, register_architecture, unregister_architecture
    from vt_transformer_b200.models.qwen2 import qwen2_model_spec
    from vt_transformer_b200.parts import unregister_part
    from vt_transformer_b200.weights import write_random_model
    Routed, Angles = define_toy_routed_parts()
    step = 0.013

    def spec(cfg):
        base = qwen2_model_spec(cfg)
        blocks = list(base.blocks)
        blocks[0] = replace(blocks[0], ffn=Routed(hidden=cfg.hidden_size, inter=40, experts=3), ffn_prefix="moe.")
        att = blocks[1].mixer
        blocks[1] = replace(blocks[1], mixer=replace(att, position=Angles(dim=att.head_dim, max_positions=cfg.max_position_embeddings,
                                                                          step=step)))
        return replace(base, blocks=tuple(blocks))

    register_architecture("ToyRoutedLM", Qwen2Config, spec, replace=True)
    try:
        d = copy.deepcopy(helpers.CONFIGS["A"])
        d["architectures"] = ["ToyRoutedLM"]
        folder = write_random_model(config_from_dict(d), os.path.join(tmp, "routed"), seed=5, sigma=0.3)
        cfg, w = plain.read_config(folder), plain.read_weights(folder)
        assert "model.layers.0.moe.experts.2.w2.weight" in w and "model.layers.0.mlp.gate_proj.weight" not in w

        def reference(ids):
            T = len(ids)
            cos, sin = plain.rotation_table(cfg.max_pos, cfg.head_dim, cfg.theta)
            x = plain.embed(w["model.embed_tokens.weight"], ids)
            # layer 0: attention as it is, then the routed feed-forward
            p = "model.layers.0."
            h = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps)
            q = plain.rotate(plain.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, cfg.heads, cfg.head_dim), range(T), cos, sin)
            k, v = plain.layer_keys_values(cfg, w, 0, x, cos, sin)
            x = x + plain.linear(plain.attention(q, k, v, None).reshape(T, -1), w[p + "self_attn.o_proj.weight"])
            h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.eps)
            prob = torch.softmax(h @ w[p + "moe.router.weight"].t(), dim=-1)
            weight, choice = prob.max(dim=-1)
            margin = float((prob.topk(2, dim=-1).values[:, 0] - prob.topk(2, dim=-1).values[:, 1]).min())
            f = torch.zeros_like(x)
            for t in range(T):
                e = int(choice[t])
                mid = plain.linear(h[t:t + 1], w[p + f"moe.experts.{e}.w1.weight"])
                f[t] = (plain.linear(mid * torch.sigmoid(mid), w[p + f"moe.experts.{e}.w2.weight"]) * weight[t])[0]
            x = x + f
            # layer 1: rotation by the other angles
            half = cfg.head_dim // 2
            angle = torch.arange(cfg.max_pos, dtype=torch.float64)[:, None] * (step * torch.arange(1, half + 1, dtype=torch.float64))[None, :]
            x = plain.layer(cfg, w, 1, x, torch.cos(angle), torch.sin(angle))
            x = plain.rms_norm(x, w["model.norm.weight"], cfg.eps)
            head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
            return plain.linear(x, head), margin

        runner = runner_for(folder, device, dtype, num_pages=12, max_requests=2)
        assert not runner.model.graph_safe()              # the routed part loops on the host: no graphs for this model
        ids = helpers.prompts_for("A")[3][:60]
        ref, margin = reference(ids)
        assert margin > (1e-4 if dtype == "float32" else 2e-2), f"a router decision is too close to call ({margin})"
        worst = 0.0
        for sizes in ([60], [7, 2, 30, 1, 1, 19], [40] + [1] * 20):
            row = runner.admit()
            got, at = [], 0
            for k in sizes:
                got.append(runner.step([helpers_entry(row, ids[at:at + k])]).float().cpu())
                at += k
            runner.check_status()
            runner.release(row)
            err = float((torch.cat(got).double() - ref).abs().max())
            # the toy rounds its experts' intermediate results and the weighted output to bfloat16 itself, at weights
            # of sigma 0.3: measured 0.57 at a spread of the logits of 2.5 (32-bit: 3.2e-5)
            assert err <= helpers.tol(dtype, ref=ref) * (1.0 if dtype == "float32" else 3.0), (sizes, err)
            worst = max(worst, err)
        return worst
    finally:
        unregister_architecture("ToyRoutedLM")
        unregister_part("feed_forward", "toy_routed")
        unregister_part("position", "toy_linear_angles")


# ----------------------------------------------------------------------------- another norm, a cache kind, the model's two ends


def define_toy_seam_parts():
    """A norm that is no RMS norm and knows nothing of a product's unadded shares (it centres the row and has a
    bias), and a mixer with a cache kind of its own: it keeps a narrow latent for every token in pages and answers
    with the mean of the latents so far.  Defined here, registered through the public registries."""
    from vt_transformer_b200.parts import (Mixer, MixerSpec, Norm, NormSpec, PagedLayout, ParamSpec, register_cache_kind,
                                           register_part)

    @dataclass(frozen=True)
    class CentredSpec(NormSpec):
        kind: str = "toy_centred"

    class Centred(Norm):
        def param_specs(self):
            return {self.prefix + ".weight": ParamSpec((self.spec.size,), role="vector", init="one_plus_normal"),
                    self.prefix + ".bias": ParamSpec((self.spec.size,), role="vector")}

        def load(self, get):
            self.w = self.rt.param(get(self.prefix + ".weight"), "vector")
            self.b = self.rt.param(get(self.prefix + ".bias"), "vector")

        def __call__(self, x, delta=None, rows=None, status=None):
            if delta is not None:
                assert isinstance(delta, torch.Tensor) and delta.shape == x.shape     # never a product's shares
                x += delta.float()
            v = x if rows is None else x[rows.long()]
            return ((v - v.mean(dim=-1, keepdim=True)) * self.w + self.b).to(self.rt.dtype)

    @dataclass(frozen=True)
    class LatentCacheSpec:
        width: int

    @dataclass(frozen=True)
    class LatentSpec(MixerSpec):
        hidden: int = 0
        width: int = 8
        kind: str = "toy_latent_memory"

    class LatentMemory(Mixer):
        def cache_spec(self):
            return LatentCacheSpec(self.spec.width)

        def param_specs(self):
            s = self.spec
            return {self.prefix + "down.weight": ParamSpec((s.width, s.hidden)),
                    self.prefix + "up.weight": ParamSpec((s.hidden, s.width))}

        def load(self, get):
            self.down = self.rt.param(get(self.prefix + "down.weight")).float()
            self.up = self.rt.param(get(self.prefix + "up.weight")).float()

        def forward(self, h, ctx, cache):
            z = cache.pages["z"]                                   # [pages, 1, page_size, width]
            out = torch.empty_like(h)
            for i, s in enumerate(ctx.seqs):
                new = h[s.offset:s.offset + s.length].float() @ self.down.t()
                end = s.start + s.length
                pos = torch.arange(end, device=h.device)
                page = cache.block_table[i, pos // cache.page_size].long()
                z[page[s.start:], 0, pos[s.start:] % cache.page_size] = new.to(z.dtype)
                mean = torch.cumsum(z[page, 0, pos % cache.page_size].float(), dim=0)[s.start:] / (pos[s.start:, None] + 1)
                out[s.offset:s.offset + s.length] = (mean @ self.up.t()).to(h.dtype)
            return out

    register_part("norm", "toy_centred", Centred, replace=True)
    register_part("mixer", "toy_latent_memory", LatentMemory, replace=True)
    register_cache_kind(LatentCacheSpec, lambda spec: PagedLayout((("z", 1, spec.width),), None))
    return CentredSpec, LatentSpec, LatentCacheSpec


def toy_seams_case(tmp, device, dtype):
    """An architecture whose embedding is scaled and whose logits are scaled and capped (fields of the model's
    spec), whose second layer's first norm and whose last norm are the toy norm, and whose second layer's mixer
    keeps latents in pages of its own kind: registered from here, built from a folder, stepped whole, in portions
    beside another request and token by token, with so few pages that they are used again."""
    from vt_transformer_b200.config import Qwen2Config, config_from_dict, register_architecture, unregister_architecture
    from vt_transformer_b200.models.qwen2 import qwen2_model_spec
    from vt_transformer_b200.parts import unregister_cache_kind, unregister_part
    from vt_transformer_b200.weights import write_random_model
    Centred, Latent, LatentCache = define_toy_seam_parts()
    scale, logit_scale, cap, width = 3.0, 3.0, 1.5, 8

    def spec(cfg):
        base = qwen2_model_spec(cfg)
        blocks = list(base.blocks)
        blocks[1] = replace(blocks[1], norm1=Centred(size=cfg.hidden_size, eps=0.0),
                            mixer=Latent(hidden=cfg.hidden_size, width=width), mixer_prefix="memory.")
        return replace(base, blocks=tuple(blocks), embedding=replace(base.embedding, scale=scale),
                       head=replace(base.head, norm=Centred(size=cfg.hidden_size, eps=0.0), logit_scale=logit_scale,
                                    logit_cap=cap))

    register_architecture("ToySeamsLM", Qwen2Config, spec, replace=True)
    try:
        d = copy.deepcopy(helpers.CONFIGS["B"])
        d["architectures"] = ["ToySeamsLM"]
        folder = write_random_model(config_from_dict(d), os.path.join(tmp, "seams"), seed=12, sigma=0.05)
        cfg, w = plain.read_config(folder), plain.read_weights(folder)
        assert "model.layers.1.memory.down.weight" in w and "model.norm.bias" in w

        def centred(x, name):
            return (x - x.mean(dim=-1, keepdim=True)) * w[name + ".weight"] + w[name + ".bias"]

        def reference(ids):
            cos, sin = plain.rotation_table(cfg.max_pos, cfg.head_dim, cfg.theta)
            x = plain.embed(w["model.embed_tokens.weight"], ids) * scale
            x = plain.layer(cfg, w, 0, x, cos, sin)
            h = centred(x, "model.layers.1.input_layernorm")
            z = h @ w["model.layers.1.memory.down.weight"].t()
            mean = torch.cumsum(z, 0) / torch.arange(1, len(ids) + 1, dtype=z.dtype)[:, None]
            x = x + mean @ w["model.layers.1.memory.up.weight"].t()
            h = plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], cfg.eps)
            x = x + plain.swiglu(h, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"],
                                 w["model.layers.1.mlp.down_proj.weight"])
            x = plain.layer(cfg, w, 2, x, cos, sin)
            logits = plain.linear(centred(x, "model.norm"), w["lm_head.weight"]) * logit_scale
            return cap * torch.tanh(logits / cap)

        runner = runner_for(folder, device, dtype, num_pages=9, max_requests=2)
        slots = runner.model.cache_slots()
        assert isinstance(slots[1], LatentCache) and len(runner.cache.groups) == 2     # keys and values; latents
        assert runner.cache.bytes_per_token() == (2 * 2 * 32 + width) * (4 if dtype == "float32" else 2)
        prompts = helpers.prompts_for("B")
        worst = 0.0
        for first, second in ((prompts[3], prompts[2]), (prompts[2], prompts[1])):   # the second pair uses rows and pages again
            rows = [runner.admit(), runner.admit()]
            got, done = [[], []], [0, 0]
            sizes = [[9, 2, 30, 1, 1, 27], [5, 1, 1, 13, 11]]
            for step in range(6):
                entries = []
                for i, ids in enumerate((first, second)):
                    if step < len(sizes[i]) and done[i] < len(ids):
                        k = min(sizes[i][step], len(ids) - done[i])
                        entries.append((i, helpers_entry(rows[i], ids[done[i]:done[i] + k])))
                        done[i] += k
                logits = runner.step([e for _, e in entries]).float().cpu()
                at = 0
                for i, e in entries:
                    got[i].append(logits[at:at + len(e.tokens)])
                    at += len(e.tokens)
            runner.check_status()
            for i, ids in enumerate((first, second)):
                assert done[i] == len(ids)
                ref = reference(ids)
                assert float(ref.abs().max()) > 0.8 * cap > float(ref.abs().median())       # the cap bends some logits, not all
                err = float((torch.cat(got[i]).double() - ref).abs().max())
                assert err <= helpers.tol(dtype, ref=ref), (i, err)
                worst = max(worst, err)
            for r in rows:
                runner.release(r)
            runner.cache.check()
        assert runner.cache.free_pages() == [9, 9]
        return worst
    finally:
        unregister_architecture("ToySeamsLM")
        unregister_part("norm", "toy_centred")
        unregister_part("mixer", "toy_latent_memory")
        unregister_cache_kind(LatentCache)


# ----------------------------------------------------------------------------- generation


def plain_generate(folder, prompt, n, temperature=0.0, seed=0, top_k=-1, top_p=1.0) -> List[int]:
    cfg, w = plain.read_config(folder), helpers._plain_weights(folder)
    from vt_transformer_b200.sampling import uniform   # the draw's random number is part of the request, not of the model
    ids = list(prompt)
    for i in range(n):
        logits = plain.forward(cfg, w, ids)[-1]
        ids.append(plain.sample(logits, temperature, uniform(seed, i), top_k, top_p))
    return ids[len(prompt):]


def greedy_generation_case(folder, name, device, dtype, n_new=16):
    """Greedy generation through the entry point.  In 32-bit the tokens are the plain
    implementation's.  In bfloat16 two logits closer than the rounding may change places, so
    each token is checked along the engine's own path: it is the plain argmax, or its plain
    logit lies within the tolerance of the largest."""
    from vt_transformer_b200 import LLM, SamplingParams
    prompts = helpers.prompts_for(name)[:3]
    llm = LLM(folder, dtype=dtype, device=device, max_running_reqs=3, num_pages=24, max_seq_len=160, page_size=16,
              max_extend_tokens=48, chunk_size=24)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert len(o) == n_new
        if dtype == "float32":
            assert o == plain_generate(folder, p, n_new), (len(p), o)
        else:
            ref = helpers.plain_logits(folder, list(p) + o)
            for i, tok in enumerate(o):
                row = ref[len(p) - 1 + i]
                assert float(row.max() - row[tok]) <= 2 * helpers.tol(dtype, name), (len(p), i, tok)
    llm.runner.cache.check()
    assert llm.stats["free_pages"] == [24] * len(llm.runner.cache.groups)
    return outs


def temperature_generation_case(folder, name, device, dtype, n_new=24):
    """Temperature sampling with a fixed seed under four settings of token budget, portion
    size and pool, the last two with so few pages that requests are pre-empted.  In 32-bit
    all settings give the plain implementation's tokens.  In bfloat16 every token is checked
    along its own path against the plain probabilities: the draw's random number falls into
    the token's interval of the plain cumulative distribution, give or take the tolerance."""
    from vt_transformer_b200 import LLM, SamplingParams
    from vt_transformer_b200.sampling import uniform
    prompts = helpers.prompts_for(name)[:4]
    params = SamplingParams(temperature=0.7, max_tokens=n_new, ignore_eos=True, seed=77)
    results, preemptions = [], []
    for kw in (dict(max_running_reqs=4, num_pages=40, max_extend_tokens=256, chunk_size=None),
               dict(max_running_reqs=4, num_pages=40, max_extend_tokens=28, chunk_size=24),
               dict(max_running_reqs=4, num_pages=11, max_extend_tokens=40, chunk_size=24),
               dict(max_running_reqs=2, num_pages=9, max_extend_tokens=16, chunk_size=5)):
        llm = LLM(folder, dtype=dtype, device=device, max_seq_len=160, page_size=16, **kw)
        results.append(llm.generate(prompts, params))
        preemptions.append(llm.stats["preemptions"])
        llm.runner.cache.check()
    assert max(preemptions) > 0, "no setting ran out of pages: the test does not test pre-emption"
    if dtype == "float32":
        for other in results[1:]:
            assert other == results[0]
        for i, (p, o) in enumerate(zip(prompts, results[0])):
            assert o == plain_generate(folder, p, n_new, temperature=0.7, seed=77 + i), i
    else:
        slack = 4 * helpers.tol(dtype, name)
        for res in results:
            for i, (p, o) in enumerate(zip(prompts, res)):
                ref = helpers.plain_logits(folder, list(p) + o)
                for j, tok in enumerate(o):
                    c = torch.cumsum(plain.kept_probabilities(ref[len(p) - 1 + j], 0.7), 0)
                    u = uniform(77 + i, j)
                    lo = float(c[tok - 1]) if tok > 0 else 0.0
                    assert lo - slack <= u <= float(c[tok]) + slack, (i, j, tok, u, lo, float(c[tok]))
    assert len({tuple(o) for o in results[0]}) > 1
    return results[0], preemptions


# ----------------------------------------------------------------------------- the next step enqueued early


def check_tokens_along_their_path(folder, prompt, out, temperature, seed, dtype, name):
    """Every generated token against the plain implementation run over the engine's own tokens: greedy, its
    plain logit lies within the tolerance of the largest; with a temperature, the draw's random number falls
    into the token's interval of the plain cumulative distribution, give or take the tolerance."""
    from vt_transformer_b200.sampling import uniform
    ref = helpers.plain_logits(folder, list(prompt) + list(out))
    for j, tok in enumerate(out):
        row = ref[len(prompt) - 1 + j]
        if temperature <= 0.0:
            assert float(row.max() - row[tok]) <= 2 * helpers.tol(dtype, name), (len(prompt), j, tok)
        else:
            c = torch.cumsum(plain.kept_probabilities(row, temperature), 0)
            u, slack = uniform(seed, j), 4 * helpers.tol(dtype, name)
            lo = float(c[tok - 1]) if tok > 0 else 0.0
            assert lo - slack <= u <= float(c[tok]) + slack, (len(prompt), j, tok, u, lo, float(c[tok]))


def overlap_generation_case(folder, name, device, dtype, n_new=24):
    """Generation with the next step enqueued before the tokens of the one before are read gives the tokens
    of generation without: greedy and with a temperature, with requests that stop at an end token (found only
    when their step lands, one step after they have run on), at their length, at different times, with
    portions of prompts between decode steps, and with so few pages that requests are pre-empted."""
    from vt_transformer_b200 import LLM, SamplingParams
    prompts = helpers.prompts_for(name)[:4]
    steps_with_overlap = 0
    for kw in (dict(max_running_reqs=4, num_pages=40, max_extend_tokens=256, chunk_size=None),
               dict(max_running_reqs=2, num_pages=40, max_extend_tokens=28, chunk_size=24),
               dict(max_running_reqs=4, num_pages=11, max_extend_tokens=40, chunk_size=24)):
        for temperature in (0.0, 0.7):
            base = SamplingParams(temperature=temperature, max_tokens=n_new, ignore_eos=True, seed=5)
            plain_llm = LLM(folder, dtype=dtype, device=device, max_seq_len=160, page_size=16, **kw)
            want = plain_llm.generate(prompts, base)
            # end tokens taken from what the requests generate: request i stops at its token number 3 + 4 i
            # (or earlier, if the same id comes earlier), the last one runs to its length
            params, stops = [], []
            for i, o in enumerate(want):
                if i == len(want) - 1:
                    params.append(SamplingParams(temperature=temperature, max_tokens=n_new - 5, ignore_eos=True, seed=5 + i))
                    stops.append(n_new - 5)
                else:
                    eos = o[min(3 + 4 * i, len(o) - 1)]
                    params.append(SamplingParams(temperature=temperature, max_tokens=n_new, seed=5 + i, eos_token_ids=(eos,)))
                    stops.append(o.index(eos) + 1)
            outs = {}
            for overlap in (False, True):
                llm = LLM(folder, dtype=dtype, device=device, max_seq_len=160, page_size=16, overlap=overlap, **kw)
                launched = []
                if overlap:
                    ahead = llm.scheduler._launch_ahead
                    def counting(flight, ahead=ahead, launched=launched):
                        got = ahead(flight)
                        launched.append(got is not None)
                        return got
                    llm.scheduler._launch_ahead = counting
                outs[overlap] = llm.generate(prompts, params)
                llm.runner.cache.check()
                assert llm.stats["free_pages"] == [kw["num_pages"]] * len(llm.runner.cache.groups)
                assert not llm.scheduler.has_work()
                steps_with_overlap += sum(launched)
            if dtype == "float32":
                assert outs[True] == outs[False], (kw, temperature)
                for o, w, n in zip(outs[False], want, stops):
                    assert o == w[:n], (kw, temperature)
            else:
                # In bfloat16 a logit may differ in its last place with the company in the batch, and the company
                # differs (a request that has ended runs one step on, others have left earlier): every token is
                # checked along its own path, and every request has stopped where its own rule says.
                for res in outs.values():
                    for i, (p, o, sp) in enumerate(zip(prompts, res, params)):
                        check_tokens_along_their_path(folder, p, o, temperature, sp.seed, dtype, name)
                        if sp.eos_token_ids and sp.eos_token_ids[0] in o:
                            assert o.index(sp.eos_token_ids[0]) == len(o) - 1, (kw, temperature, i)
                        else:
                            assert len(o) == sp.max_tokens, (kw, temperature, i)
    assert steps_with_overlap > 20, "hardly a step was enqueued early: the test does not test it"


# ----------------------------------------------------------------------------- real layer widths, wide steps

_models = {}


def shared_runner(folder, device, dtype, num_pages, max_requests=4, max_seq_len=None, page_size=16):
    """A runner over a model that is loaded once for each (folder, dtype) and shared: the model folders of real
    widths hold gigabytes.  The cache manager, and with it the pool, the block tables and the captured graphs,
    is the runner's own."""
    from vt_transformer_b200.cache.manager import CacheManager
    from vt_transformer_b200.engine.runner import ModelRunner
    key = (folder, str(device), dtype)
    if key not in _models:
        base = ModelRunner.from_folder(folder, dtype=dtype, device=device, page_size=16, num_pages=1, max_requests=1,
                                       max_seq_len=16)
        _models[key] = (base.model, base.rt)
    model, rt = _models[key]
    if max_seq_len is None:
        max_seq_len = model.spec.max_positions
    cache = CacheManager(model.cache_slots(), page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                         max_seq_len=max_seq_len, dtype=rt.dtype, device=rt.device)
    return ModelRunner(model, cache, rt)


def forget_shared_models():
    _models.clear()


def replay_family_shared(folder, name, family, device, dtype, n_prompts=4, sizes=None, page_size=16):
    """``replay_family`` for a model of real widths: the first ``n_prompts`` requests, the model shared."""
    prompts = helpers.prompts_for(name)[:n_prompts]
    make = {"whole": helpers.trace_whole, "tail": helpers.trace_tail,
            "portions": (lambda p: helpers.trace_portions(p, sizes=sizes)) if sizes else helpers.trace_portions,
            "mixed": lambda p: helpers.trace_mixed(p, max_live=4, seed=3)}[family]
    trace = make(prompts)
    pages = helpers.tokens_needed(trace, round_to=page_size) // page_size
    runner = shared_runner(folder, device, dtype, num_pages=pages, page_size=page_size)
    got = helpers.run_trace_inproc(runner, trace)
    worst = helpers.compare_trace(folder, prompts, trace, got, helpers.tol(dtype, name))
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.groups]
    return worst


def wide_decode_case(folder, name, device, dtype, sequences, decode_steps, runner=None, page_size=16, budget=512,
                     bound=None):
    """Decode steps of many live requests.  ``sequences``: token lists of different lengths.  Each request's
    tokens but the last ``decode_steps`` run as prompt portions (several requests a step, up to ``budget`` tokens);
    then every request brings one token a step, all in one step, and every row of logits is compared with the
    plain implementation.  Returns (worst difference, the graph keys (batch bucket, context bucket) that ran)."""
    from vt_transformer_b200.engine.batch import StepEntry
    n = len(sequences)
    if runner is None:
        pages = sum(-(-len(s) // page_size) for s in sequences)
        runner = shared_runner(folder, device, dtype, num_pages=pages, max_requests=n, page_size=page_size)
    rows = [runner.admit() for _ in range(n)]
    done = [0] * n
    heads = [max(1, len(s) - decode_steps) for s in sequences]
    while any(d < h for d, h in zip(done, heads)):
        entries, left = [], budget
        for i in range(n):
            if done[i] < heads[i] and left > 0:
                k = min(heads[i] - done[i], left)
                entries.append(StepEntry(rows[i], sequences[i][done[i]:done[i] + k], []))
                done[i] += k
                left -= k
        runner.step(entries)
    worst, bound = 0.0, (helpers.tol(dtype, name) if bound is None else bound)
    for step in range(decode_steps):
        live = [i for i in range(n) if done[i] < len(sequences[i])]
        if not live:
            break
        logits = runner.step([StepEntry(rows[i], [sequences[i][done[i]]], [0]) for i in live]).double().cpu()
        runner.check_status()
        for j, i in enumerate(live):
            ref = helpers.plain_logits(folder, sequences[i])[done[i]]
            d = float((logits[j] - ref).abs().max())
            assert d == d and d <= bound, (f"decode step {step} of {len(live)} requests: request {i} (length "
                                          f"{len(sequences[i])}) at position {done[i]}: |dlogit| {d:.3e} > {bound:.1e}")
            worst = max(worst, d)
            done[i] += 1
    keys = sorted({k[:2] for k in runner._graphs})      # (batch bucket, bound of the cached lengths)
    for r in rows:
        runner.release(r)
    runner.cache.check()
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.groups]
    return worst, keys
