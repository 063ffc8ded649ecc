"""The CPU reference execution: a model folder run whole, in float32, by the host runtime's plain
C++ loops (``hi_b200/csrc/host/cpu_forward.cpp``): no GPU, no cache, no kernels of the serving
path. It is what ``python -m hi_b200 run --cpu`` uses (the reference's
``--execution cpu-reference``: crates/hi-cuda/src/lib.rs:205-226, crates/hi-cuda/src/qwen_cpu.rs:84-261)
and the second plain statement of the formulas that the test-suite's own plain model is held
against. It takes the same typed configuration, registry, loader and parts' tensors as the
engine; what it computes with them is its own.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..config.registry import load_architecture
from ..host import build as host
from ..parts.attention import AttentionMixer
from ..parts.basic import LinearHead, NoPosition, RMSNorm, RotaryPosition, TokenEmbedding
from ..parts.feed_forward import DenseSwiGLU, SigmoidRoutedExperts
from ..parts.model import Model
from ..weights.loader import load_from_dir

F, I, P = ctypes.c_float, ctypes.c_int, ctypes.c_void_p


class _CpuModel(ctypes.Structure):
    _fields_ = [("hidden", I), ("vocab", I), ("final_eps", F), ("embedding", P), ("final_norm", P), ("head", P)]


class _CpuLayer(ctypes.Structure):
    _fields_ = [("mixer", I), ("heads", I), ("kv_heads", I), ("head_dim", I), ("chunk", I), ("sliding", I),
                ("interleaved", I), ("qk_norm", I), ("temperature", I), ("scale", F), ("qk_eps", F), ("floor_scale", F),
                ("attn_scale", F), ("norm_eps", F), ("inv_freq", P), ("rot_pairs", I), ("norm_mixer", P), ("norm_feed_forward", P),
                ("wq", P), ("wk", P), ("wv", P), ("wo", P), ("bq", P), ("bk", P), ("bv", P), ("bo", P),
                ("feed_forward", I), ("inter", I), ("experts", I), ("top_k", I), ("shared_inter", I),
                ("w_gate", P), ("w_up", P), ("w_down", P), ("router", P), ("shared_gate", P), ("shared_up", P),
                ("shared_down", P), ("forced_ids", P)]


class CpuReference:
    """A loaded model and its whole-sequence float32 forward on the CPU."""

    def __init__(self, model: Model):
        if model.dtype != torch.float32 or model.device.type != "cpu" or not model.loaded:
            raise ValueError("the CPU reference takes a loaded float32 model on the CPU")
        self.model = model
        self._keep: List[np.ndarray] = []
        self._lib = host.library()
        emb, head, norm = model.embedding, model.head, model.final_norm
        for part, kind in ((emb, TokenEmbedding), (head, LinearHead), (norm, RMSNorm)):
            if not isinstance(part, kind):
                raise ValueError(f"the CPU reference does not know the part {type(part).__name__}")
        table = self._f32(emb.table)
        self._model = _CpuModel(hidden=model.spec.hidden_size, vocab=model.spec.vocab_size, final_eps=norm.eps,
                                embedding=table.ctypes.data, final_norm=self._f32(norm.weight).ctypes.data,
                                head=(table if head.weight is None else self._f32(head.weight)).ctypes.data)
        self._layers = (_CpuLayer * len(model.layers))(*[self._layer(l) for l in model.layers])
        self.schedule = np.asarray([e.layer for e in model.spec.schedule], dtype=np.int32)
        self.routed_names = [f"{model.layers[e.layer].feed_forward.prefix}" for e in model.spec.schedule
                             if isinstance(model.layers[e.layer].feed_forward, SigmoidRoutedExperts)]
        self.top_k = {l.feed_forward.prefix: l.feed_forward.top_k for l in model.layers
                      if isinstance(l.feed_forward, SigmoidRoutedExperts)}

    @staticmethod
    def from_dir(model_dir: str) -> "CpuReference":
        arch, cfg, _raw = load_architecture(model_dir)
        model = Model(arch.build_spec(cfg), torch.float32, "cpu")
        load_from_dir(model, model_dir, arch.normalize_tensor_name, arch.derive_tensors)
        return CpuReference(model)

    def _f32(self, t: Optional[torch.Tensor]) -> Optional[np.ndarray]:
        if t is None:
            return None
        a = np.ascontiguousarray(t.detach().to(torch.float32).cpu().numpy())
        self._keep.append(a)
        return a

    def _ptr(self, t: Optional[torch.Tensor]):
        a = self._f32(t)
        return None if a is None else a.ctypes.data

    def _layer(self, layer) -> _CpuLayer:
        mix, ff = layer.mixer, layer.feed_forward
        if not isinstance(mix, AttentionMixer) or not isinstance(layer.norm_mixer, RMSNorm) or \
                not isinstance(layer.norm_feed_forward, RMSNorm) or layer.spec.arrangement != "prenorm":
            raise ValueError(f"the CPU reference does not know the parts of {layer.spec.prefix}")
        if layer.norm_mixer.eps != layer.norm_feed_forward.eps:
            raise ValueError(f"{layer.spec.prefix}: the CPU reference takes one eps for both norms of a layer")
        nh, nkv, hd = mix.nh, mix.nkv, mix.hd
        wq, wk, wv = mix.w_qkv.split([nh * hd, nkv * hd, nkv * hd], dim=0)
        bq = bk = bv = None
        if mix.b_qkv is not None:
            bq, bk, bv = mix.b_qkv.split([nh * hd, nkv * hd, nkv * hd], dim=0)
        inv_freq, interleaved = None, False
        if isinstance(mix.position, RotaryPosition):
            inv_freq, interleaved = torch.from_numpy(mix.position._table_host), mix.position.interleaved
        elif not isinstance(mix.position, NoPosition):
            raise ValueError(f"the CPU reference does not know the position part {type(mix.position).__name__}")
        window = mix.window or (None, 0)
        L = _CpuLayer(mixer=1, heads=nh, kv_heads=nkv, head_dim=hd, chunk=window[1] if window[0] == "chunk" else 0,
                      sliding=window[1] if window[0] == "sliding" else 0, interleaved=int(interleaved),
                      qk_norm=int(mix.qk_norm), temperature=int(mix.temperature is not None), scale=mix.scale,
                      qk_eps=mix.qk_norm_eps, floor_scale=(mix.temperature or (1.0, 0.0))[0],
                      attn_scale=(mix.temperature or (1.0, 0.0))[1], norm_eps=layer.norm_mixer.eps,
                      inv_freq=self._ptr(inv_freq), rot_pairs=0 if inv_freq is None else int(inv_freq.numel()), norm_mixer=self._ptr(layer.norm_mixer.weight),
                      norm_feed_forward=self._ptr(layer.norm_feed_forward.weight), wq=self._ptr(wq), wk=self._ptr(wk),
                      wv=self._ptr(wv), wo=self._ptr(mix.w_o), bq=self._ptr(bq), bk=self._ptr(bk), bv=self._ptr(bv),
                      bo=self._ptr(mix.b_o))
        if isinstance(ff, DenseSwiGLU):
            gate, up = ff.mlp.w_gate_up.split(ff.mlp.inter, dim=0)
            L.feed_forward, L.inter = 1, ff.mlp.inter
            L.w_gate, L.w_up, L.w_down = self._ptr(gate), self._ptr(up), self._ptr(ff.mlp.w_down)
        elif isinstance(ff, SigmoidRoutedExperts):
            if ff.router_mode or ff.scale_output:
                raise ValueError(f"{layer.spec.prefix}: the CPU reference knows sigmoid scores on the experts' input only")
            L.feed_forward, L.inter, L.experts, L.top_k = 2, ff.inter, ff.experts, ff.top_k
            L.w_gate, L.w_up, L.w_down, L.router = (self._ptr(ff.w_gate), self._ptr(ff.w_up), self._ptr(ff.w_down),
                                                    self._ptr(ff.w_router))
            if ff.shared is not None:
                gate, up = ff.shared.w_gate_up.split(ff.shared.inter, dim=0)
                L.shared_inter = ff.shared.inter
                L.shared_gate, L.shared_up, L.shared_down = self._ptr(gate), self._ptr(up), self._ptr(ff.shared.w_down)
        else:
            raise ValueError(f"the CPU reference does not know the feed-forward part {type(ff).__name__}")
        return L

    def forward(self, tokens: Sequence[int], want: Optional[Sequence[int]] = None,
                forced_routing: Optional[Dict[str, torch.Tensor]] = None, return_routing: bool = False):
        """float32 logits [len(want), vocab] (every position when ``want`` is None) of one sequence.
        ``forced_routing`` {feed-forward prefix: ids [T, k]} replaces those layers' expert choices;
        ``return_routing`` adds {prefix: ids [T, k]} of the choices taken (the last run of a layer
        that the schedule names twice)."""
        toks = np.asarray(list(tokens), dtype=np.int32)
        T = int(toks.size)
        rows = np.arange(T, dtype=np.int32) if want is None else np.asarray(list(want), dtype=np.int32)
        logits = np.empty((rows.size, self._model.vocab), dtype=np.float32)
        keep = []
        for i, layer in enumerate(self.model.layers):
            ids = (forced_routing or {}).get(layer.feed_forward.prefix)
            if ids is not None:
                a = np.ascontiguousarray(torch.as_tensor(ids).to(torch.int32).cpu().numpy().reshape(T, -1))
                keep.append(a)
                self._layers[i].forced_ids = a.ctypes.data
            else:
                self._layers[i].forced_ids = None
        if return_routing and len(set(self.top_k.values())) > 1:
            raise ValueError("return_routing needs the same top_k in every routed layer")
        k = next(iter(self.top_k.values()), 1)
        chosen = np.empty((max(len(self.routed_names), 1), T, k), dtype=np.int32)     # [routed entry, token, rank]
        code = self._lib.hbh_cpu_forward(ctypes.byref(self._model), self._layers, self.schedule.ctypes.data,
                                         int(self.schedule.size), toks.ctypes.data, T, rows.ctypes.data, int(rows.size),
                                         logits.ctypes.data, chosen.ctypes.data if return_routing else None)
        if code != 0:
            raise ValueError(f"the CPU reference refused its input (code {code}): token ids outside the vocabulary, "
                             "positions outside the sequence, or forced expert ids outside the experts")
        out = torch.from_numpy(logits)
        if not return_routing:
            return out
        return out, {name: torch.from_numpy(chosen[i].copy()) for i, name in enumerate(self.routed_names)}

    def generate(self, tokens: Sequence[int], max_tokens: int, params=None, eos_token_ids: Sequence[int] = ()) -> List[int]:
        """Generation by running the whole sequence again for every token (no cache): greedy, or
        sampled by the host sampler's rule with the request's generator."""
        from ..sampling.sampler import DEFAULT_SEED, Lcg, SamplingParams, sample_on_host

        params = params or SamplingParams(max_tokens=max_tokens)
        rng = Lcg(DEFAULT_SEED if params.seed is None else params.seed)
        seq, out = list(tokens), []
        stops = set(eos_token_ids) if not params.ignore_eos else set()
        stops |= set(params.stop_token_ids or ())
        for _ in range(max_tokens):
            row = self.forward(seq, want=[len(seq) - 1])[0].numpy()
            tok = sample_on_host(row, params, rng)
            if tok in stops:
                break
            out.append(tok)
            seq.append(tok)
        return out
