"""Tusipel: a pre-norm decoder whose sublayers read a short convolution of the normalised stream, over two kinds of attention and
dense or routed feed-forwards, with a repeated span of layers.

``config.json`` lists the layers one by one (``layers[i] = {type, mixer, mlp}``).  The embedding is multiplied by
``embedding.scale``; a block is :class:`ConvPreNormDecoderLayer` (``x <- x + mixer(c(norm1(x)))``, ``x <- x + mlp(c(norm2(x)))`` with
``c(h) = h + causal_conv(h)`` over ``canon.taps`` positions, norm weights stored around zero).  Parts:

* mixer ``latent_attention`` — :class:`LatentSinkAttention` configured with a query latent, a rotated key part shared by the heads
  (rotate-half layout, YaRN-scaled frequencies), a sliding window and a sigmoid gate per output channel; the cache holds the
  normalised latent row and the rotated part, nothing else;
* mixer ``attention`` — :class:`ConvWindowAttention` configured without biases, row norms, rotation or gate: grouped-query attention
  over convolved q / k / v, a distance term ``slope_h (i - j)`` taken off the scores, keys visible inside the query's chunk only;
* feed-forward ``dense`` — :class:`ClampedGLUMLP`; ``moe`` — :class:`MoE`: softmax router whose choice uses corrected scores among the
  best groups of experts, gated SiLU experts, identity experts behind the last router outputs, weights scaled and not renormalised;
* ``loop`` — layers ``start .. stop-1`` run ``times`` times in a row with the same weights; every run has caches and carried rows of
  its own, and the embedding output is added to the stream right before every pass but the first;
* output: final norm, head.

Every size and constant comes from the checkpoint's ``config.json``.  The engine side is the one the other hybrid stacks use: the
paged cache with per-run shapes (:class:`LayeredBlockKVCacheManager`), state lines for everything carried per sequence, ragged rows
(prompt portions beside single decoded tokens) in one forward, decode steps replayed from CUDA graphs.
"""
from __future__ import annotations

import json
import math
import os
from typing import List

import torch
import torch.nn as nn

from ... import ops
from ...config import InferenceConfig, NeuronConfig
from ...modules.attention.conv_window_attention import ConvWindowAttention
from ...modules.attention.latent_attention import LatentSinkAttention
from ...modules.kvcache import LayeredBlockKVCacheManager
from ...modules.mlp import ClampedGLUMLP
from ...modules.moe import ExpertMLPs, MoE, RouterTopK
from ...modules.norm import RMSNorm
from ...modules.rope import compute_inv_freq
from ...modules.sampling import Sampler
from ...parallel.layers import ColumnParallelLinear, ParallelEmbedding
from ..application_base import NeuronBaseForCausalLM
from ..model_base import ConvPreNormDecoderLayer, NeuronBaseModel
from ..sodudra.modeling_sodudra import layer_runs

GLU_ALPHA = 1.702        # slope of the sigmoid in the dense feed-forward's gate product (fixed by the design)
YARN_MAGNITUDE = 0.1     # cos / sin are multiplied by YARN_MAGNITUDE * ln(factor) + 1


def rope_of(rot: dict):
    """(inverse frequencies fp64 [dims / 2], magnitude of cos / sin, cache tag) of a mixer's ``rot`` entry."""
    dims, base, sc = int(rot["dims"]), float(rot["base"]), rot.get("scaling")
    if not sc:
        inv, mag = compute_inv_freq(dims, base, None, dtype=torch.float64)
        return inv, 1.0, ("plain", dims, base)
    factor = float(sc["factor"])
    mag = YARN_MAGNITUDE * math.log(factor) + 1.0
    inv, _ = compute_inv_freq(dims, base, dict(rope_type="yarn", factor=factor, original_max_position_embeddings=sc["original"],
                                               beta_fast=sc["fast"], beta_slow=sc["slow"], attention_factor=mag), dtype=torch.float64)
    return inv, mag, ("yarn", dims, base, factor, sc["original"], sc["fast"], sc["slow"])


class TusipelInferenceConfig(InferenceConfig):
    def get_required_attributes(self) -> List[str]:
        return ["layers", "norm", "vocab", "width"]

    def add_derived_config(self):
        self.num_cores_per_group = 1
        self.hidden_size, self.vocab_size, self.num_hidden_layers = self.width, self.vocab, len(self.layers)
        self.rms_norm_eps = float(self.norm["eps"])
        for name, default in (("loop", None), ("canon", None), ("embedding", None)):
            if not hasattr(self, name):
                setattr(self, name, default)
        self.canon_taps = int((self.canon or {}).get("taps") or 0)
        self.embedding_scale = float((self.embedding or {}).get("scale", 1.0))
        for i, layer in enumerate(self.layers):
            if layer["type"] not in ("latent_attention", "attention"):
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown mlp kind {mlp.get('kind')!r}")
            if layer["type"] == "latent_attention":
                m = layer["mixer"]
                if int(m.get("rot_dim") or 0) and int(m["rot"]["dims"]) != int(m["rot_dim"]):
                    raise ValueError(f"layer {i}: the rotation covers the whole rotated part (rot.dims == rot_dim)")
        self.runs = layer_runs(len(self.layers), self.loop)

    @classmethod
    def get_neuron_config_cls(cls):
        return NeuronConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig) -> "TusipelInferenceConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            d = json.load(f)

        def load(self):
            for k, v in d.items():
                setattr(self, k, v)
        return cls(neuron_config, load_config=load)


class NeuronTusipelModel(NeuronBaseModel):
    meta_extra_keys = ("computed_context_lens",)
    graph_tensor_kwargs = ("slot_mapping", "block_table", "computed_context_lens", "gather_positions")

    def __init__(self, config, device=None):
        super().__init__(config, device)
        # every op of a step is a sync-free kernel launch or a torch op on static shapes (the routed experts run on a device-side
        # permutation with a static row bound); rows with seq_id -1 have q_len 0 and touch neither cache nor state
        self.graph_safe = device is not None and torch.device(device).type == "cuda"

    def setup_attr_for_model(self, config):
        nc = config.neuron_config
        if nc.tp_degree != 1:
            raise NotImplementedError("Tusipel: tensor parallel degree 1")
        if not nc.is_block_kv_layout:
            raise ValueError("Tusipel runs on the paged KV cache: set is_block_kv_layout=True, pa_block_size, pa_num_blocks")
        self.tp_degree, self.hidden_size = 1, config.width
        self.max_batch_size, self.buckets = nc.max_batch_size, nc.buckets

    def _mixer(self, i, spec, W, eps, dt, dev):
        m = spec["mixer"]
        mask = (m.get("mask") or {}).get("size")
        scale = float(m["scale"]) if m.get("scale") is not None else m["dim"] ** -0.5
        if spec["type"] == "latent_attention":
            rot = int(m.get("rot_dim") or 0)
            return LatentSinkAttention(W, m["heads"], m["dim"], m.get("vdim", m["dim"]), m["kv_rank"], scale=scale, eps=eps, sink=False,
                                       head_gate=False, layer_idx=i, dtype=dt, device=dev, tp_group=self.tp_group,
                                       q_rank=int(m.get("q_rank") or 0), rot_dim=rot, rope=rope_of(m["rot"]) if rot else None, window=mask,
                                       channel_gate=True)
        return ConvWindowAttention(W, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"]),
                                   conv_taps=int(m.get("conv") or 1), rot_dims=0, rot_base=1.0, scale=scale, softcap=None, window=None,
                                   keep_first=0, eps=eps, layer_idx=i, dtype=dt, device=dev, tp_group=self.tp_group, bias=False,
                                   row_norm=False, out_gate=False, chunk=mask, distance_bias=True)

    def _mlp(self, f, W, dt, dev):
        if f is None:
            return None
        if f["kind"] == "dense":
            return ClampedGLUMLP(W, f["ff"], f["limit"], GLU_ALPHA, dt, self.tp_group, dev)
        r = f["router"]
        ident = int(r.get("identity") or 0)
        g = r.get("groups")
        router = RouterTopK(r["experts"] + ident, r["top"], W, dt, "softmax", False, False, False, dev, correction=True,
                            groups=(g["count"], g["keep"]) if g else None, scale=float(r.get("scale", 1.0)))
        experts = ExpertMLPs(r["experts"], W, f["expert"]["ff"], "silu", dt, False, dev)
        return MoE(router, experts, None, identity_experts=ident)

    def init_model(self, config):
        nc = config.neuron_config
        dev, dt = self.device_, nc.torch_dtype
        W, eps = config.width, config.rms_norm_eps
        self.embed_tokens = ParallelEmbedding(config.vocab, W, None, dtype=dt, device=dev, shard_across_embedding=True, pad=True,
                                              tensor_model_parallel_group=self.tp_group)
        norm = lambda: RMSNorm(W, eps, torch.float32, device=dev)       # noqa: E731  (the loader stores 1 + w)
        layers = []
        for i, spec in enumerate(config.layers):
            mlp = self._mlp(spec.get("mlp"), W, dt, dev)
            layers.append(ConvPreNormDecoderLayer(self._mixer(i, spec, W, eps, dt, dev), mlp, norm(), norm() if mlp is not None else None,
                                                  W, config.canon_taps, i, dev))
        self.layers = nn.ModuleList(layers)
        self.runs = list(config.runs)
        self.norm = norm()
        self.lm_head = ColumnParallelLinear(W, config.vocab, bias=False, gather_output=False, dtype=dt, device=dev, pad=True,
                                            tensor_model_parallel_group=self.tp_group)

    def _kernels_cover_decode(self) -> bool:
        return False

    def init_inference_optimization(self, config):
        nc = self.neuron_config
        if self.on_device_sampling:
            self.sampler = Sampler(nc, self.tp_group, vocab_shard=False)
        # caches and carried rows per layer RUN: a layer of the repeated span sees different streams in different passes
        shapes, specs = {}, {}
        for r, (i, _) in enumerate(self.runs):
            shapes[r] = self.layers[i].mixer.kv_shape()
            specs.update(self.layers[i].state_specs(r))
        self.kv_mgr = LayeredBlockKVCacheManager(shapes, {}, nc.pa_num_blocks, nc.pa_block_size, nc.torch_dtype, self.device_,
                                                 state_specs=specs, num_slots=nc.kv_cache_batch_size, state_dtype=nc.torch_dtype)

    # ---- forward hooks ---------------------------------------------------------------------------------------------------
    def build_meta(self, input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw):
        meta = super().build_meta(input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw)
        if meta.block_table is None:
            raise ValueError("Tusipel: every forward needs block_table (paged KV cache)")
        B, T = input_ids.shape[:2]
        dev = input_ids.device
        q_len = meta.key_valid.sum(-1).to(torch.int32) if meta.key_valid is not None else torch.full((B,), T, dtype=torch.int32, device=dev)
        q_len = torch.where(meta.seq_ids < 0, torch.zeros_like(q_len), q_len)
        ctx = meta.extras.get("computed_context_lens")
        ctx = meta.position_ids[:, 0] if ctx is None else ctx.to(dev)
        meta.extras.update(q_len=q_len.contiguous(), ctx_len=ctx.to(torch.int32).contiguous(),
                           state_lines=self.kv_mgr.lines_for(meta.seq_ids).to(torch.int32).contiguous(),
                           act_dtype=self.neuron_config.torch_dtype)
        return meta

    def embed(self, input_ids, inputs_embeds=None, vision_embeddings=None, vision_mask=None):
        h = super().embed(input_ids, inputs_embeds, vision_embeddings, vision_mask).float()      # fp32 residual stream
        return h * self.config.embedding_scale if self.config.embedding_scale != 1.0 else h

    def run_layers(self, emb, meta):
        x, pending = emb, None
        for r, (i, t) in enumerate(self.runs):
            x, pending = self.layers[i](x, pending, meta, self.kv_mgr, r, extra=emb if t else None)     # passes after the first re-read the embedding
            if meta.capture is not None:
                meta.capture[f"runs.{r}.out"] = x + pending.float()
        return ops.stream_add_rmsnorm(x, (pending,))[0]          # the last sublayer's output joins the stream

    def _finish(self, h, lp_dtype=None):
        return ops.stream_add_rmsnorm(h.float(), weight=self.norm.weight, eps=self.norm.variance_epsilon, lp_dtype=lp_dtype)[2]

    def final_hidden(self, h):
        return self._finish(h)

    def compute_logits(self, h):
        return self.lm_head(self._finish(h, self.neuron_config.torch_dtype))


class NeuronTusipelForCausalLM(NeuronBaseForCausalLM):
    _model_cls = NeuronTusipelModel
    _STATE_DICT_MODEL_PREFIX = ""

    @classmethod
    def get_config_cls(cls):
        return TusipelInferenceConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig):
        return cls(model_path, TusipelInferenceConfig.from_pretrained(model_path, neuron_config))

    @staticmethod
    def convert_hf_to_neuron_state_dict(sd: dict, config) -> dict:
        """Checkpoint names (``l<i>.mix.q`` ...) -> module parameters: the projections that read the same input stacked for one GEMM,
        the up-projections viewed per head, the experts' matrices stacked along a leading expert axis, norm weights as ``1 + w``."""
        one_plus = lambda w: 1.0 + w.float()          # noqa: E731
        out = {"embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"], "norm.weight": one_plus(sd["final.norm"])}
        for i, spec in enumerate(config.layers):
            a, b = f"l{i}.", f"layers.{i}."
            out[b + "norm1.weight"] = one_plus(sd[a + "norm1"])
            if a + "canon1" in sd:
                out[b + "conv1_weight"] = sd[a + "canon1"]
            x, y, m = a + "mix.", b + "mixer.", spec["mixer"]
            if spec["type"] == "latent_attention":
                H, R = m["heads"], m["kv_rank"]
                first = sd[x + "dq"] if m.get("q_rank") else sd[x + "q"]
                out[y + "in_proj.weight"] = torch.cat([first, sd[x + "dkv"], sd[x + "g"]], 0)
                if m.get("q_rank"):
                    out[y + "q_norm_weight"] = sd[x + "dq.norm"]
                    out[y + "q_up.weight"] = sd[x + "uq"]
                out[y + "latent_norm_weight"] = sd[x + "dkv.norm"]
                out[y + "k_up"] = sd[x + "uk"].reshape(H, m["dim"], R)
                out[y + "v_up"] = sd[x + "uv"].reshape(H, m.get("vdim", m["dim"]), R)
            else:
                out[y + "in_proj.weight"] = torch.cat([sd[x + n] for n in ("q", "k", "v")], 0)
                ident = lambda n: torch.ones(sd[x + n].shape[0], 1, dtype=sd[x + n].dtype)          # noqa: E731  (no convolution: one tap of one)
                out[y + "conv_weight"] = torch.cat([sd.get(x + n + ".conv", ident(n)) for n in ("q", "k", "v")], 0)
            out[y + "o_proj.weight"] = sd[x + "o"]
            f = spec.get("mlp")
            if f is None:
                continue
            out[b + "norm2.weight"] = one_plus(sd[a + "norm2"])
            if a + "canon2" in sd:
                out[b + "conv2_weight"] = sd[a + "canon2"]
            x, y = a + "mlp.", b + "mlp."
            if f["kind"] == "dense":
                out[y + "gate_up_proj.weight"] = torch.cat([sd[x + "gate"], sd[x + "up"]], 0)
                out[y + "down_proj.weight"] = sd[x + "down"]
            else:
                E = f["router"]["experts"]
                out[y + "router.linear_router.weight"] = sd[x + "router"]
                out[y + "router.score_correction"] = sd[x + "correction"]
                out[y + "expert_mlps.gate_up_proj"] = torch.stack([torch.cat([sd[f"{x}e{e}.gate"], sd[f"{x}e{e}.up"]], 0) for e in range(E)], 0)
                out[y + "expert_mlps.down_proj"] = torch.stack([sd[f"{x}e{e}.down"] for e in range(E)], 0)
        return out

    def init_random_weights(self, seed: int = 0):
        """Benchmarks: N(0, 0.02) projections, unit norms, small convolution taps, no score correction."""
        super().init_random_weights(seed)
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                if name.endswith(("norm1.weight", "norm2.weight", "norm_weight")) or name == "norm.weight":
                    p.fill_(1.0)
                elif name.endswith(("conv1_weight", "conv2_weight")):
                    p.fill_(0.1)
                elif name.endswith("conv_weight"):
                    p.fill_(1.0 / p.shape[1])
                elif name.endswith("score_correction"):
                    p.zero_()
