"""Zanivik: a decoder whose blocks are normalised on both sides of every sublayer and whose mixers are PAIRS, an attention layer and a
recurrent layer side by side on the same input.

``config.json`` lists the layers one by one (``layers[i] = {type, mixer: {left, right, ...}, mlp}``).  A block is
:class:`SandwichNormDecoderLayer`: ``r = mixer(norm1(x))``, ``x += m * ls1 * norm1b(r)``, then ``r = mlp(norm2(x))``, ``x += m * ls2 * norm2b(r)`` with
``m = residual_mult``, layer norms without bias and learned layer scales.  Mixer types (:class:`SideBySideMixer`):

* ``parallel`` — left :class:`HeadNormWindowAttention` with rotate-half rotary positions (optionally Llama-3-scaled frequencies), q / k
  divided by their per-head root mean square AFTER the rotation (no weight), a sliding window, a sink in the softmax denominator and a
  sigmoid output gate; right :class:`RaggedGatedDeltaMixer`; result ``left_scale * left + right_scale * right``;
* ``parallel_2`` — left :class:`HeadNormWindowAttention` without a value projection (the raw key slice doubles as the value), weighted
  per-head q / k norms BEFORE the rotation, a learned temperature per head and a sliding window; right :class:`RaggedMamba2Mixer`;
  result ``0.5 * (rms_unit(left) * w_left + rms_unit(right) * w_right)`` with the RMS norms over the model width.

Feed-forward: ``W_down gelu(W_up h)`` with the exact (erf) GELU (:class:`PlainMLP`).  Output: final layer norm, head.  Every size and
constant comes from the checkpoint's ``config.json``.  The engine side is the one the other hybrid stacks use: the paged cache with
per-layer shapes (:class:`LayeredBlockKVCacheManager`) for the attention halves, state lines for convolution tails and recurrent
states, ragged rows (prompt portions beside single decoded tokens) in one forward, decode steps replayed from CUDA graphs.
"""
from __future__ import annotations

import json
import os
from typing import List

import torch
import torch.nn as nn

from ...config import InferenceConfig, NeuronConfig
from ...modules.attention.head_norm_window_attention import HeadNormWindowAttention
from ...modules.attention.side_by_side import SideBySideMixer
from ...modules.kvcache import LayeredBlockKVCacheManager
from ...modules.mlp import PlainMLP
from ...modules.norm import LayerNorm
from ...modules.sampling import Sampler
from ...modules.ssm import RaggedGatedDeltaMixer, RaggedMamba2Mixer
from ...parallel.layers import ColumnParallelLinear, ParallelEmbedding
from ..application_base import NeuronBaseForCausalLM
from ..model_base import NeuronBaseModel, SandwichNormDecoderLayer

MIXER_TYPES = ("parallel", "parallel_2")


class ZanivikInferenceConfig(InferenceConfig):
    def get_required_attributes(self) -> List[str]:
        return ["layers", "norm", "vocab", "width"]

    def add_derived_config(self):
        self.num_cores_per_group = 1
        self.hidden_size, self.vocab_size, self.num_hidden_layers = self.width, self.vocab, len(self.layers)
        self.rms_norm_eps = float(self.norm["eps"])
        if not hasattr(self, "residual_mult"):
            self.residual_mult = 1.0
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown mlp kind {mlp.get('kind')!r}")
            left = layer["mixer"]["left"]
            if layer["type"] == "parallel_2" and left.get("vdim", left["dim"]) != left["dim"]:
                raise ValueError(f"layer {i}: values that are the keys have the keys' size")

    @classmethod
    def get_neuron_config_cls(cls):
        return NeuronConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig) -> "ZanivikInferenceConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            d = json.load(f)

        def load(self):
            for k, v in d.items():
                setattr(self, k, v)
        return cls(neuron_config, load_config=load)


class NeuronZanivikModel(NeuronBaseModel):
    meta_extra_keys = ("computed_context_lens",)
    graph_tensor_kwargs = ("slot_mapping", "block_table", "computed_context_lens", "gather_positions")

    def __init__(self, config, device=None):
        super().__init__(config, device)
        # every op of a step is a sync-free kernel launch or a torch op on static shapes; rows with seq_id -1 have q_len 0 and touch
        # neither cache nor state
        self.graph_safe = device is not None and torch.device(device).type == "cuda"

    def setup_attr_for_model(self, config):
        nc = config.neuron_config
        if nc.tp_degree != 1:
            raise NotImplementedError("Zanivik: tensor parallel degree 1")
        if not nc.is_block_kv_layout:
            raise ValueError("Zanivik runs on the paged KV cache: set is_block_kv_layout=True, pa_block_size, pa_num_blocks")
        self.tp_degree, self.hidden_size = 1, config.width
        self.max_batch_size, self.buckets = nc.max_batch_size, nc.buckets

    def _mixer(self, i, spec, W, eps, dt, dev):
        m = spec["mixer"]
        L, R = m["left"], m["right"]
        rot, mask = L.get("rot") or {}, (L.get("mask") or {}).get("size")
        kw = dict(rot_dims=int(rot.get("dims") or 0), rot_base=float(rot.get("base") or 10000.0), rot_scaling=rot.get("scaling"),
                  scale=float(L["scale"]) if L.get("scale") is not None else L["dim"] ** -0.5, window=mask, eps=eps, layer_idx=i,
                  own_in_proj=False, dtype=dt, device=dev, tp_group=self.tp_group)
        heads, kv = L["heads"], L.get("kv_heads", L["heads"])
        taps = int(R.get("conv") or 1)
        if spec["type"] == "parallel":
            left = HeadNormWindowAttention(W, heads, kv, L["dim"], L.get("vdim", L["dim"]), norm_at="post", norm_weight=False, sink=True,
                                           out_gate=True, **kw)
            right = RaggedGatedDeltaMixer(W, R["heads"], R.get("kv_heads", R["heads"]), R["dim"], R.get("vdim", R["dim"]), taps, eps, i,
                                          dtype=dt, device=dev, tp_group=self.tp_group, own_in_proj=False)
            return SideBySideMixer(W, left, right, left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)),
                                   dtype=dt, device=dev, tp_group=self.tp_group)
        left = HeadNormWindowAttention(W, heads, kv, L["dim"], L["dim"], norm_at="pre", norm_weight=True, head_temp=True, value_from_key=True, **kw)
        right = RaggedMamba2Mixer(W, R["heads"], R["vdim"], R["state"], int(R.get("groups") or 1), int(R.get("norm_groups") or 1), taps, eps, i,
                                  dtype=dt, device=dev, tp_group=self.tp_group, own_in_proj=False)
        return SideBySideMixer(W, left, right, left_scale=0.5, right_scale=0.5, out_norm=True, dtype=dt, device=dev, tp_group=self.tp_group)

    def init_model(self, config):
        nc = config.neuron_config
        dev, dt = self.device_, nc.torch_dtype
        W, eps = config.width, config.rms_norm_eps
        self.embed_tokens = ParallelEmbedding(config.vocab, W, None, dtype=dt, device=dev, shard_across_embedding=True, pad=True,
                                              tensor_model_parallel_group=self.tp_group)
        norm = lambda: LayerNorm(W, eps, bias=False, dtype=torch.float32, device=dev)       # noqa: E731
        layers = []
        for i, spec in enumerate(config.layers):
            f = spec.get("mlp")
            mlp = PlainMLP(W, f["ff"], "gelu", dt, False, self.tp_group, dev) if f is not None else None
            layers.append(SandwichNormDecoderLayer(self._mixer(i, spec, W, eps, dt, dev), mlp, norm(), norm(), norm() if f is not None else None,
                                                   norm() if f is not None else None, W, float(config.residual_mult), True, i, dev))
        self.layers = nn.ModuleList(layers)
        self.norm = norm()
        self.lm_head = ColumnParallelLinear(W, config.vocab, bias=False, gather_output=False, dtype=dt, device=dev, pad=True,
                                            tensor_model_parallel_group=self.tp_group)

    def _kernels_cover_decode(self) -> bool:
        return False

    def init_inference_optimization(self, config):
        nc = self.neuron_config
        if self.on_device_sampling:
            self.sampler = Sampler(nc, self.tp_group, vocab_shard=False)
        shapes, specs = {}, {}
        for i, layer in enumerate(self.layers):
            shapes[i] = layer.mixer.kv_shape()
            specs.update(layer.state_specs())
        self.kv_mgr = LayeredBlockKVCacheManager(shapes, {}, nc.pa_num_blocks, nc.pa_block_size, nc.torch_dtype, self.device_,
                                                 state_specs=specs, num_slots=nc.kv_cache_batch_size, state_dtype=nc.torch_dtype)

    # ---- forward hooks ---------------------------------------------------------------------------------------------------
    def build_meta(self, input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw):
        meta = super().build_meta(input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw)
        if meta.block_table is None:
            raise ValueError("Zanivik: every forward needs block_table (paged KV cache)")
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
        return super().embed(input_ids, inputs_embeds, vision_embeddings, vision_mask).float()      # fp32 residual stream

    def run_layers(self, x, meta):
        pending = None
        for i, layer in enumerate(self.layers):
            x, pending = layer(x, pending, meta, self.kv_mgr)
            if meta.capture is not None:
                meta.capture[f"layers.{i}.out"] = SandwichNormDecoderLayer.finish(x, pending)[0]
        return SandwichNormDecoderLayer.finish(x, pending)[0]          # the last sublayer's output joins the stream

    def _finish(self, h, lp_dtype=None):
        return SandwichNormDecoderLayer.finish(h.float(), None, self.norm.weight, self.norm.eps, True, lp_dtype)[1]

    def final_hidden(self, h):
        return self._finish(h)

    def compute_logits(self, h):
        return self.lm_head(self._finish(h, self.neuron_config.torch_dtype))


class NeuronZanivikForCausalLM(NeuronBaseForCausalLM):
    _model_cls = NeuronZanivikModel
    _STATE_DICT_MODEL_PREFIX = ""

    @classmethod
    def get_config_cls(cls):
        return ZanivikInferenceConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig):
        return cls(model_path, ZanivikInferenceConfig.from_pretrained(model_path, neuron_config))

    @staticmethod
    def convert_hf_to_neuron_state_dict(sd: dict, config) -> dict:
        """Checkpoint names (``l<i>.mix.left.q`` ...) -> module parameters; the projections of both mixers of a pair that read the
        block's input are stacked ``[left | right]`` for one GEMM, the three short convolutions of the gated delta rule likewise."""
        out = {"embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"], "norm.weight": sd["final.norm"]}
        for i, spec in enumerate(config.layers):
            a, b = f"l{i}.", f"layers.{i}."
            for n in ("norm1", "norm1b"):
                out[b + n + ".weight"] = sd[a + n]
            out[b + "ls1"] = sd[a + "ls1"]
            x, y = a + "mix.", b + "mixer."
            lx, rx, ly, ry = x + "left.", x + "right.", y + "left.", y + "right."
            if spec["type"] == "parallel":
                left = [sd[lx + n] for n in ("q", "k", "v", "g")]
                right = [sd[rx + n] for n in ("q", "k", "v", "b", "a", "g")]
                out[ly + "sinks"] = sd[lx + "sink"]
                taps = int(spec["mixer"]["right"].get("conv") or 1)
                ident = lambda n: torch.ones(sd[rx + n].shape[0], 1, dtype=sd[rx + n].dtype)          # noqa: E731  (no convolution: one tap of one)
                out[ry + "conv_weight"] = torch.cat([sd[rx + n + ".conv"] if taps > 1 or (rx + n + ".conv") in sd else ident(n) for n in ("q", "k", "v")], 0)
                for src, dst in (("A_log", "A_log"), ("dt_bias", "dt_bias"), ("norm", "norm_weight"), ("o", "out_proj.weight")):
                    out[ry + dst] = sd[rx + src]
            else:
                left = [sd[lx + n] for n in ("q", "k")]
                right = [sd[rx + "in"]]
                out[ly + "q_norm_weight"], out[ly + "k_norm_weight"], out[ly + "head_temp"] = sd[lx + "q.norm"], sd[lx + "k.norm"], sd[lx + "temp"]
                out[y + "left_out_weight"], out[y + "right_out_weight"] = sd[lx + "out"], sd[rx + "out"]
                for src, dst in (("conv", "conv_weight"), ("conv.b", "conv_bias"), ("dt_bias", "dt_bias"), ("A_log", "A_log"), ("D", "D"),
                                 ("norm", "norm_weight"), ("o", "out_proj.weight")):
                    if rx + src in sd:
                        out[ry + dst] = sd[rx + src]
                if rx + "conv" not in sd:
                    m = spec["mixer"]["right"]
                    cd = m["heads"] * m["vdim"] + 2 * int(m.get("groups") or 1) * m["state"]
                    out[ry + "conv_weight"] = torch.ones(cd, 1, dtype=sd[rx + "in"].dtype)
            out[y + "in_proj.weight"] = torch.cat(left + right, 0)
            out[ly + "o_proj.weight"] = sd[lx + "o"]
            if spec.get("mlp") is not None:
                for n in ("norm2", "norm2b"):
                    out[b + n + ".weight"] = sd[a + n]
                out[b + "ls2"] = sd[a + "ls2"]
                out[b + "mlp.fc1.weight"], out[b + "mlp.fc2.weight"] = sd[a + "mlp.up"], sd[a + "mlp.down"]
        return out

    def init_random_weights(self, seed: int = 0):
        """Benchmarks: N(0, 0.02) projections; norms, scales, decays and step biases at values that keep the stream well scaled."""
        super().init_random_weights(seed)
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                if name.endswith(("norm1.weight", "norm2.weight", "norm1b.weight", "norm2b.weight", "norm_weight", "out_weight", "head_temp", ".D", "ls1", "ls2")) \
                        or name == "norm.weight":
                    p.fill_(1.0)
                elif name.endswith("conv_weight"):
                    p.fill_(1.0 / p.shape[1])
                elif name.endswith(("A_log", "sinks", "conv_bias")):
                    p.zero_()
                elif name.endswith("dt_bias"):
                    p.fill_(-2.0)
