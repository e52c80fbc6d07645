"""MoEConfig / Router / MoELayer with the reference's call API (src/core/), running on
libmoe_b200's CUDA kernels.

    config = create_moe_config(num_experts=8, expert_type="gated", input_dim=512, hidden_dim=2048,
                               output_dim=512, activation=silu, gate_type=TopKGating(2),
                               balance_loss=SwitchTransformerLoss(0.01))
    moe = MoELayer(config)
    output, balance_loss = moe(x, training=True)        # x: (input_dim, T), output: (output_dim, T)

Matrices keep the reference's shapes.  Julia stores (input_dim x T) column-major, i.e. T
contiguous token vectors; pass ``x_TD.t()`` (torch) or an F-ordered NumPy array to avoid a copy.
CUDA tensors run in place on torch's current stream; NumPy arrays go through the host entry
point (copy in, compute, copy out).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np

from . import _lib
from . import experts as _experts
from .experts import GatedExpert, StandardExpert
from .gating import GatingMechanism, SharedExpertGating, SwitchGating, TopKGating, gate_kind_of
from .losses import AuxiliaryFreeLoss, LoadBalancingLoss, SwitchTransformerLoss


@dataclass
class MoEConfig:
    """Base.@kwdef struct MoEConfig (src/core/moe_layer.jl:4-29), same fields and defaults."""
    num_experts: int = 8
    expert_type: str = "standard"
    input_dim: int = 768
    hidden_dim: int = 3072
    output_dim: int = 768
    activation: Callable = _experts.gelu
    expert_dropout: float = 0.0
    gate_type: GatingMechanism = field(default_factory=lambda: TopKGating(2))
    top_k: int = 2                      # not read by the forward pass (k comes from gate_type)
    noise_scale: float = 0.0
    use_noise_network: bool = False
    use_fp32_router: bool = True
    balance_loss: LoadBalancingLoss = field(default_factory=lambda: SwitchTransformerLoss(0.01))
    z_loss_weight: float = 0.001
    capacity_factor: float = 1.25
    drop_tokens: bool = False
    use_cur: bool = False
    cur_rank: Optional[int] = None
    num_shared_experts: int = 0


def create_moe_config(**kwargs) -> MoEConfig:
    """create_moe_config(; kwargs...) (src/core/moe_layer.jl:281-283)."""
    return MoEConfig(**kwargs)


_ACT_PROBE = np.array([-3.0, -1.0, -0.25, 0.0, 0.5, 2.0], dtype=np.float64)


def activation_enum(fn) -> int:
    """Map MoEConfig.activation (any callable in the reference) to the C ABI's enum: by
    identity for the functions this package exports, else by probing the callable on a few
    points.  Anything else is refused - there is no CPU path to run an arbitrary function."""
    if isinstance(fn, str):
        table = {"silu": _lib.ACT_SILU, "swish": _lib.ACT_SILU, "gelu": _lib.ACT_GELU_TANH,
                 "relu": _lib.ACT_RELU, "identity": _lib.ACT_IDENTITY}
        if fn in table:
            return table[fn]
        raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"unknown activation '{fn}'")
    known = [(_experts.silu, _lib.ACT_SILU), (_experts.gelu, _lib.ACT_GELU_TANH),
             (_experts.relu, _lib.ACT_RELU), (_experts.identity, _lib.ACT_IDENTITY)]
    for f, e in known:
        if fn is f:
            return e
    try:
        got = np.array([float(fn(float(v))) for v in _ACT_PROBE])
    except Exception as exc:  # noqa: BLE001
        raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"activation {fn!r} cannot be probed: {exc}") from exc
    for f, e in known:
        if np.allclose(got, f(_ACT_PROBE), rtol=1e-5, atol=1e-6):
            return e
    raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"activation {fn!r} is not one of silu/gelu/relu/identity")


class Router:
    """Router (src/core/router.jl:4-23): a bias-free (num_experts x input_dim) projection with
    Flux's default Glorot-uniform init, plus the gate that turns logits into assignments."""

    def __init__(self, input_dim: int, num_experts: int, gate_type: GatingMechanism, *, noise_scale: float = 0.0,
                 use_noise_network: bool = False, use_fp32: bool = True, rng=None):
        g = rng if isinstance(rng, np.random.Generator) else np.random.default_rng(rng)
        lim = math.sqrt(6.0 / (input_dim + num_experts))
        self.weight = g.uniform(-lim, lim, size=(num_experts, input_dim)).astype(np.float32)
        self.noise_weight = None
        self.gate_type = gate_type
        self.noise_scale = float(noise_scale)
        self.use_fp32 = bool(use_fp32)
        if use_noise_network:    # a second Dense(input_dim, num_experts, bias=false) (src/core/router.jl:20)
            self.noise_weight = g.uniform(-lim, lim, size=(num_experts, input_dim)).astype(np.float32)


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _weight_ptr_layout(w):
    """(pointer, dtype enum, layout enum, is_device, keepalive) of an (out, in) weight."""
    if _is_torch(w):
        import torch

        if w.dtype == torch.float32:
            dt = _lib.DTYPE_F32
        elif w.dtype == torch.bfloat16:
            dt = _lib.DTYPE_BF16
        else:
            raise _lib.MoEError(_lib.ERR_INVALID, f"unsupported weight dtype {w.dtype}")
        if w.is_contiguous():
            return w.data_ptr(), dt, _lib.LAYOUT_IN_CONTIG, int(w.is_cuda), w
        if w.t().is_contiguous():
            return w.data_ptr(), dt, _lib.LAYOUT_OUT_CONTIG, int(w.is_cuda), w
        wc = w.contiguous()
        return wc.data_ptr(), dt, _lib.LAYOUT_IN_CONTIG, int(wc.is_cuda), wc
    a = np.asarray(w)
    if a.dtype != np.float32:
        a = a.astype(np.float32)
    if a.flags.c_contiguous:
        return a.ctypes.data, _lib.DTYPE_F32, _lib.LAYOUT_IN_CONTIG, 0, a
    if a.flags.f_contiguous:
        return a.ctypes.data, _lib.DTYPE_F32, _lib.LAYOUT_OUT_CONTIG, 0, a
    a = np.ascontiguousarray(a)
    return a.ctypes.data, _lib.DTYPE_F32, _lib.LAYOUT_IN_CONTIG, 0, a


class _HostValue:
    """A host result with the two accessors the lazy statistics use on device tensors."""

    def __init__(self, v):
        self.v = v

    def cpu(self):
        return self

    def numpy(self):
        return np.asarray(self.v)

    def item(self):
        return float(self.v)


class _BoundForward:
    """One forward call with its arguments bound (MoELayer.bind_forward)."""

    def __init__(self, layer, xt, out, T, training):
        import torch

        self._layer, self._xt, self.out, self.T, self.training = layer, xt, out, T, training
        dev = xt.device
        self.loss = torch.zeros((), dtype=torch.float32, device=dev)
        self.tokens_per_expert = torch.zeros(layer.config.num_experts, dtype=torch.int64, device=dev)
        self.routing_entropy = torch.zeros((), dtype=torch.float32, device=dev)
        o = _lib.ForwardOutputs()
        o.loss = self.loss.data_ptr()
        o.tokens_per_expert, o.routing_entropy = self.tokens_per_expert.data_ptr(), self.routing_entropy.data_ptr()
        self._o = o
        self._args = (xt.data_ptr(), _lib.DTYPE_BF16 if xt.dtype == torch.bfloat16 else _lib.DTYPE_F32, T, int(training),
                      out.data_ptr(), C.byref(o))
        self._device = dev
        self._current_stream = torch.cuda.current_stream

    def __call__(self):
        rc = _lib.lib.moe_layer_forward(self._layer._handle, *self._args, self._current_stream(self._device).cuda_stream)
        if rc:
            _lib.check(rc)
        return self.out.t(), self.loss


class MoELayer:
    """MoELayer(config) (src/core/moe_layer.jl:34-63) and its call
    ``moe(x; training=false, return_stats=false) -> (output, balance_loss[, training_stats])``
    (:107-128).

    Extra keywords (no counterpart in the reference): ``device`` (CUDA ordinal),
    ``compute_dtype`` ("f32": FP32 FMA path, 1e-5 parity class; "bf16": tcgen05 tensor cores),
    ``experts`` / ``router`` to inject pre-built weights, ``rng`` to seed the default init,
    ``weights_on_device`` to draw the default expert weights on the GPU, ``weight_image`` (bytes
    or a uint8 array made by ``export_weights``) to load every weight with plain copies instead:
    the layer then keeps no host copy of experts or router."""

    def __init__(self, config: MoEConfig, *, device: int = 0, compute_dtype: str = "f32", experts=None, router=None,
                 rng=None, weights_on_device: bool = False, expert_parallel=None, weight_image=None):
        self.config = config
        self.device = int(device)
        self.compute_dtype = compute_dtype
        self._handle = C.c_void_p()
        # create_experts (src/core/moe_layer.jl:65-102): :gated builds GatedExpert, anything else StandardExpert
        self.gated = str(config.expert_type).lstrip(":") == "gated"
        if not self.gated and config.expert_dropout > 0:
            raise _lib.MoEError(_lib.ERR_UNSUPPORTED, "expert_dropout > 0 (Dropout inside StandardExpert) is not accelerated")
        if config.use_cur:
            raise _lib.MoEError(_lib.ERR_UNSUPPORTED, "CUR experts are not accelerated")
        kind, k, gate_shared = gate_kind_of(config.gate_type)
        if gate_shared and config.num_shared_experts:
            raise _lib.MoEError(_lib.ERR_INVALID, "use either SharedExpertGating or num_shared_experts, not both")
        shared_mode = _lib.SHARED_GATING if gate_shared else (
            _lib.SHARED_LAYER_BLEND if config.num_shared_experts > 0 else _lib.SHARED_NONE)
        num_shared = gate_shared or config.num_shared_experts
        self.balance_loss = config.balance_loss
        if isinstance(self.balance_loss, AuxiliaryFreeLoss) and self.balance_loss.num_experts != config.num_experts:
            # update_bias! indexes its count vector with layer expert ids (auxiliary_free.jl:48-53)
            raise _lib.MoEError(_lib.ERR_INVALID, "AuxiliaryFreeLoss must be built for config.num_experts experts")
        if isinstance(self.balance_loss, AuxiliaryFreeLoss):
            alpha = self.balance_loss.complementary_weight if self.balance_loss.use_complementary_loss else 0.0
        elif isinstance(self.balance_loss, SwitchTransformerLoss):
            alpha = self.balance_loss.alpha
        else:
            raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"balance_loss {type(self.balance_loss).__name__} is not accelerated")
        self._cfg = _lib.MoeConfig(
            num_experts=config.num_experts, num_shared=num_shared, top_k=k, input_dim=config.input_dim,
            hidden_dim=config.hidden_dim, output_dim=config.output_dim, gate_kind=kind,
            activation=activation_enum(config.activation),
            compute_dtype={"f32": _lib.DTYPE_F32, "bf16": _lib.DTYPE_BF16}[compute_dtype],
            shared_mode=shared_mode, balance_alpha=float(alpha), z_loss_weight=float(config.z_loss_weight),
            index_base=1, bias_gates_only=1 if isinstance(self.balance_loss, AuxiliaryFreeLoss) else 0,
            capacity_factor=float(config.capacity_factor), drop_tokens=int(bool(config.drop_tokens)),
            expert_kind=_lib.EXPERT_GATED if self.gated else _lib.EXPERT_STANDARD)
        _lib.check(_lib.lib.moe_layer_create(C.byref(self._cfg), self.device, C.byref(self._handle)))
        kt, ep, er = C.c_int32(), C.c_int32(), C.c_int32()
        _lib.check(_lib.lib.moe_layer_dims(self._handle, C.byref(kt), C.byref(ep), C.byref(er)))
        self.k_out, self.e_probs, self.e_router = kt.value, ep.value, er.value

        self.expert_range = range(config.num_experts)
        if expert_parallel is not None:
            rank, world, uid = expert_parallel
            _lib.check(_lib.lib.moe_ep_init(self._handle, uid, int(rank), int(world)))
            per = config.num_experts // world
            self.expert_range = range(rank * per, (rank + 1) * per)

        if weight_image is not None:
            self._expert_factory, self.experts, self.router = None, [None] * config.num_experts, None
            self._stats = {"tokens_per_expert": np.zeros(config.num_experts, dtype=np.int64),
                           "routing_entropy": [], "capacity_overflow": 0}
            self._pending = []
            self._aux_on_device = False
            self.import_weights(weight_image)
            if isinstance(self.balance_loss, AuxiliaryFreeLoss):
                self._attach_aux_free(expert_parallel is not None)
            return
        if experts is None:
            dev = f"cuda:{self.device}" if weights_on_device else None
            make = GatedExpert if self.gated else StandardExpert
            experts = [make(config.input_dim, config.hidden_dim, config.output_dim, config.activation,
                            rng=rng, device=dev) if e in self.expert_range else None
                       for e in range(config.num_experts)]
        # `experts` may be a callable e -> GatedExpert: each expert is then built, copied to the
        # device and dropped, so the host (or torch) copy of a large layer never exists at once
        self._expert_factory = experts if callable(experts) else None
        self.experts = [None] * config.num_experts if callable(experts) else list(experts)
        self.router = router if router is not None else Router(
            config.input_dim, self.e_router, config.gate_type, noise_scale=config.noise_scale,
            use_noise_network=config.use_noise_network, use_fp32=config.use_fp32_router, rng=rng)
        self._stats = {"tokens_per_expert": np.zeros(config.num_experts, dtype=np.int64),
                       "routing_entropy": [], "capacity_overflow": 0}
        self._pending = []          # device-side (tokens_per_expert, entropy) of calls not yet folded in
        self._aux_on_device = False
        self.sync_weights()
        if isinstance(self.balance_loss, AuxiliaryFreeLoss):
            self._attach_aux_free(expert_parallel is not None)

    @property
    def training_stats(self) -> dict:
        """moe.training_stats (src/core/moe_layer.jl:56-60): cumulative tokens_per_expert, the
        routing entropy of every call, capacity_overflow.  Device-side results of earlier
        calls are folded in here, so a forward on CUDA tensors never waits for the GPU."""
        for tpe, ent in self._pending:
            self._stats["tokens_per_expert"] += tpe.cpu().numpy()
            self._stats["routing_entropy"].append(float(ent.item()))
        self._pending.clear()
        return self._stats

    # -- weights ---------------------------------------------------------------------------
    def export_weights(self) -> np.ndarray:
        """The layer's device-resident weights (experts, router, bias, noise network) as one uint8
        array in the library's own layout and compute dtype: what serialize_moe_layer
        (src/llama2/utils.jl:258-303) stores for a layer, ready to be loaded without repacking."""
        n = int(_lib.lib.moe_layer_weights_image_bytes(self._handle))
        if n < 0:
            raise _lib.MoEError(_lib.ERR_STATE, _lib.lib.moe_last_error().decode("utf-8", "replace"))
        img = np.empty(n, dtype=np.uint8)
        _lib.check(_lib.lib.moe_layer_export_weights(self._handle, img.ctypes.data, n))
        return img

    def import_weights(self, image) -> None:
        """Load an ``export_weights`` image made by a layer of the same configuration."""
        img = np.frombuffer(image, dtype=np.uint8) if isinstance(image, (bytes, bytearray, memoryview)) else \
            np.ascontiguousarray(image, dtype=np.uint8)
        _lib.check(_lib.lib.moe_layer_import_weights(self._handle, img.ctypes.data, img.size))

    def sync_weights(self) -> None:
        """Copy (and repack) the experts' and the router's current weights into the device
        handle; call again after mutating them."""
        if self.router is None:
            raise _lib.MoEError(_lib.ERR_STATE, "this layer was loaded from a weight image: it has no host weights to sync")
        for e in self.expert_range:
            ex = self._expert_factory(e) if self._expert_factory else self.experts[e]
            p1, d1, l1, dev1, k1 = _weight_ptr_layout(ex.w1)
            p2, d2, l2, dev2, k2 = _weight_ptr_layout(ex.w2)
            if not self.gated:
                if not (d1 == d2 and l1 == l2 and dev1 == dev2):
                    raise _lib.MoEError(_lib.ERR_INVALID, "w1, w2 of an expert must share dtype, layout and device")
                pb1, kb1 = self._bias_ptr(ex.b1, ex.hidden_dim, dev1)
                pb2, kb2 = self._bias_ptr(ex.b2, ex.output_dim, dev1)
                _lib.check(_lib.lib.moe_layer_set_expert_standard(self._handle, e, p1, pb1, p2, pb2, d1, l1, dev1))
                continue
            p3, d3, l3, dev3, k3 = _weight_ptr_layout(ex.w3)
            if not (d1 == d2 == d3 and l1 == l2 == l3 and dev1 == dev2 == dev3):
                raise _lib.MoEError(_lib.ERR_INVALID, "w1, w2, w3 of an expert must share dtype, layout and device")
            _lib.check(_lib.lib.moe_layer_set_expert(self._handle, e, p1, p2, p3, d1, l1, dev1))
        self.sync_router()

    def _attach_aux_free(self, expert_parallel: bool) -> None:
        """Move AuxiliaryFreeLoss's state into the device handle (update_bias! then runs at the end of
        every training forward on the GPU); with expert parallelism or num_shared_experts > 0 the
        update stays on the host, fed by the call's expert counts."""
        bl = self.balance_loss
        if expert_parallel or self.config.num_shared_experts > 0:
            return
        mom = np.ascontiguousarray(bl._bias_momentum, dtype=np.float32)
        _lib.check(_lib.lib.moe_layer_set_aux_free(self._handle, 1, bl.learning_rate, bl.momentum, bl.update_freq,
                                                   mom.ctypes.data, bl._update_counter))
        self._aux_on_device = True

        def state():
            n = self.e_router
            b, m_ = np.empty(n, dtype=np.float32), np.empty(n, dtype=np.float32)
            cnt = C.c_int64()
            _lib.check(_lib.lib.moe_layer_aux_free_state(self._handle, b.ctypes.data, m_.ctypes.data, C.byref(cnt)))
            return b, m_, int(cnt.value)

        def push():
            bl._device_state = None              # sync_router reads the host copy just assigned
            try:
                self.sync_router()
                mom2 = np.ascontiguousarray(bl._bias_momentum, dtype=np.float32)
                _lib.check(_lib.lib.moe_layer_set_aux_free(self._handle, 1, bl.learning_rate, bl.momentum,
                                                           bl.update_freq, mom2.ctypes.data, bl._update_counter))
            finally:
                bl._device_state = state

        bl._device_state, bl._device_push = state, push

    def _bias_ptr(self, b, n: int, on_device: int):
        """Pointer to a float32 copy of bias vector ``b`` in the memory kind of the weights."""
        if b is None:
            return None, None
        if _is_torch(b):
            import torch

            keep = b.detach().to(dtype=torch.float32).contiguous()
            keep = keep.cuda(self.device) if on_device else keep.cpu()
            ptr, size = keep.data_ptr(), keep.numel()
        elif on_device:
            import torch

            keep = torch.as_tensor(np.asarray(b, dtype=np.float32)).cuda(self.device)
            ptr, size = keep.data_ptr(), keep.numel()
        else:
            keep = np.ascontiguousarray(b, dtype=np.float32)
            ptr, size = keep.ctypes.data, keep.size
        if size != n:
            raise _lib.MoEError(_lib.ERR_INVALID, f"expert bias must have {n} entries, got {size}")
        return ptr, keep

    def sync_router(self) -> None:
        if self.router is None:
            raise _lib.MoEError(_lib.ERR_STATE, "this layer was loaded from a weight image: it has no host weights to sync")
        w = self.router.weight
        p, d, lay, dev, keep = _weight_ptr_layout(w)
        if d != _lib.DTYPE_F32:
            raise _lib.MoEError(_lib.ERR_INVALID, "router weights must be float32")
        bias_ptr, keep_b = None, None
        bias = getattr(self.router, "bias", None)
        if isinstance(self.balance_loss, AuxiliaryFreeLoss) and self.config.num_shared_experts == 0:
            # forward_standard alone selects with the biased logits (src/core/moe_layer.jl:137-140);
            # forward_with_shared_experts (:158-185) only updates the bias
            bias = self.balance_loss.bias
        if bias is not None:
            if _is_torch(bias):
                import torch

                keep_b = bias.to(dtype=torch.float32).contiguous()
                if bool(keep_b.is_cuda) != bool(dev):
                    keep_b = keep_b.cuda(self.device) if dev else keep_b.cpu()
                bias_ptr = keep_b.data_ptr()
            else:
                if dev:
                    import torch

                    keep_b = torch.as_tensor(np.asarray(bias, dtype=np.float32)).cuda(self.device)
                    bias_ptr = keep_b.data_ptr()
                else:
                    keep_b = np.ascontiguousarray(bias, dtype=np.float32)
                    bias_ptr = keep_b.ctypes.data
            n = keep_b.numel() if _is_torch(keep_b) else keep_b.size
            if n != self.e_router:
                raise _lib.MoEError(_lib.ERR_INVALID, f"router bias must have {self.e_router} entries")
        _lib.check(_lib.lib.moe_layer_set_router(self._handle, p, bias_ptr, lay, dev))
        nw = getattr(self.router, "noise_weight", None)
        if nw is not None:
            pn, dn, layn, devn, keep_n = _weight_ptr_layout(nw)
            if dn != _lib.DTYPE_F32:
                raise _lib.MoEError(_lib.ERR_INVALID, "router noise weights must be float32")
            _lib.check(_lib.lib.moe_layer_set_router_noise_network(self._handle, pn, layn, devn))
        else:
            _lib.check(_lib.lib.moe_layer_set_router_noise_network(self._handle, None, 0, 0))

    # -- forward ---------------------------------------------------------------------------
    def __call__(self, x, training: bool = False, return_stats: bool = False, return_routing: bool = False,
                 out=None, router_noise=None):
        """``out`` (optional, no counterpart in the reference): a preallocated float32 (T, output_dim)
        C-ordered buffer of the same kind as x (CUDA tensor / NumPy array, e.g. pinned) that
        receives the result; the returned output is its (output_dim, T) view.
        ``router_noise`` (optional): the standard-normal draws, shape (router rows, T), used when
        ``training`` and ``config.noise_scale > 0`` (src/core/router.jl:38-40); drawn with torch on the
        layer's device when omitted."""
        cfg = self.config
        if x.ndim != 2 or x.shape[0] != cfg.input_dim:
            raise _lib.MoEError(_lib.ERR_INVALID, f"x must have shape (input_dim={cfg.input_dim}, T), got {tuple(x.shape)}")
        T = int(x.shape[1])
        aux_free = isinstance(self.balance_loss, AuxiliaryFreeLoss) and training
        noise_keep = self._arm_router_noise(T, training, router_noise)
        want_stats = cfg.num_shared_experts == 0 or (aux_free and not self._aux_on_device)
        if _is_torch(x) and x.is_cuda:
            out, loss, extra = self._forward_torch(x, T, training, want_stats, return_routing, out)
        else:
            out, loss, extra = self._forward_host(x if _is_torch(x) else np.asarray(x), T, training, want_stats,
                                                  return_routing, out)
        if noise_keep is not None:
            _lib.check(_lib.lib.moe_layer_set_router_noise(self._handle, None, 0.0))
        if cfg.num_shared_experts == 0:
            # update_stats! (src/core/moe_layer.jl:250-264) runs in forward_standard only
            self._pending.append((extra["tokens_per_expert"], extra["routing_entropy"]))
            if len(self._pending) > 256:
                _ = self.training_stats
        if aux_free and not self._aux_on_device:
            # compute_loss(::AuxiliaryFreeLoss) updates the bias first (auxiliary_free.jl:73-83); the
            # device handle does it itself unless the configuration keeps the update on the host
            tpe = extra["tokens_per_expert"]
            tpe = np.array(tpe.cpu().numpy() if _is_torch(tpe) else tpe)
            # forward_with_shared_experts hands compute_loss the routed ids shifted past the shared
            # experts (moe_layer.jl:176-179), so those never count
            tpe[:cfg.num_shared_experts] = 0
            self.balance_loss.update_bias(tpe)
            if cfg.num_shared_experts == 0:
                self.sync_router()
        ret = (out, loss)
        if return_stats:
            ret = ret + (self.training_stats,)
        if return_routing:
            ret = ret + ({k: extra[k] for k in ("indices", "gates", "probs", "logits")},)
        return ret

    def _arm_router_noise(self, T, training, router_noise):
        """Hand the draws of this call's router noise to the device handle (a (T, rows) float32
        CUDA tensor that must stay alive until the forward has been queued)."""
        scale = float(getattr(self.router, "noise_scale", 0.0) or 0.0)
        if not training or scale <= 0.0:
            return None
        import torch

        dev = torch.device(f"cuda:{self.device}")
        if router_noise is None:
            if not hasattr(self, "_noise_gen"):
                self._noise_gen = torch.Generator(device=dev)
            nz = torch.randn((T, self.e_router), device=dev, generator=self._noise_gen, dtype=torch.float32)
        else:
            nz = torch.as_tensor(np.asarray(router_noise) if not _is_torch(router_noise) else router_noise)
            nz = nz.to(device=dev, dtype=torch.float32).t().contiguous()
            if tuple(nz.shape) != (T, self.e_router):
                raise _lib.MoEError(_lib.ERR_INVALID, f"router_noise must have shape ({self.e_router}, T)")
        torch.cuda.synchronize(dev)     # the draws are read on another stream by a host-path call
        _lib.check(_lib.lib.moe_layer_set_router_noise(self._handle, nz.data_ptr(), scale))
        return nz

    def _forward_torch(self, x, T, training, want_stats, want_routing, out=None):
        import torch

        cfg = self.config
        xt = x.t()
        if not xt.is_contiguous():
            xt = xt.contiguous()
        if xt.dtype == torch.float32:
            xd = _lib.DTYPE_F32
        elif xt.dtype == torch.bfloat16:
            xd = _lib.DTYPE_BF16
        else:
            xt = xt.float()
            xd = _lib.DTYPE_F32
        dev = xt.device
        if out is None:
            out = torch.empty((T, cfg.output_dim), dtype=torch.float32, device=dev)
        elif (tuple(out.shape) != (T, cfg.output_dim) or out.dtype != torch.float32 or not out.is_contiguous()
              or out.device != dev):
            raise _lib.MoEError(_lib.ERR_INVALID, "out must be a contiguous float32 (T, output_dim) tensor on x's device")
        # the library writes every optional output it is given on every call (zeros for an empty batch)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        o = _lib.ForwardOutputs()
        o.loss = loss.data_ptr()
        extra = {}
        if want_stats:
            tpe = torch.empty(cfg.num_experts, dtype=torch.int64, device=dev)
            ent = torch.empty((), dtype=torch.float32, device=dev)
            o.tokens_per_expert, o.routing_entropy = tpe.data_ptr(), ent.data_ptr()
        if want_routing:
            idx = torch.empty((T, self.k_out), dtype=torch.int32, device=dev)
            gates = torch.empty((T, self.k_out), dtype=torch.float32, device=dev)
            probs = torch.empty((T, self.e_probs), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.e_router), dtype=torch.float32, device=dev)
            o.indices, o.gates, o.probs, o.logits = idx.data_ptr(), gates.data_ptr(), probs.data_ptr(), logits.data_ptr()
            extra.update(indices=idx.t(), gates=gates.t(), probs=probs.t(), logits=logits.t())
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.lib.moe_layer_forward(self._handle, xt.data_ptr(), xd, T, int(training), out.data_ptr(),
                                                  C.byref(o), stream))
        if want_stats:
            extra["tokens_per_expert"] = tpe
            extra["routing_entropy"] = ent
        return out.t(), loss, extra

    def bind_forward(self, x, out, training: bool = False):
        """Bind the arguments of one device forward once and return a callable that only makes the C
        call (no counterpart in the reference: for loops whose steps are shorter than the checks and
        allocations of ``__call__``, e.g. token-by-token decoding into fixed buffers).  ``x`` is the
        (input_dim, T) view of a contiguous (T, input_dim) float32/bfloat16 CUDA tensor and ``out`` a
        contiguous float32 (T, output_dim) CUDA tensor; both are read and written in place by every
        call, on the stream that is current when the call is made.  The returned object keeps
        ``loss``, ``tokens_per_expert`` and ``routing_entropy`` tensors that every call overwrites;
        ``training_stats`` is not updated by bound calls."""
        import torch

        cfg = self.config
        xt = x.t()
        if (x.ndim != 2 or x.shape[0] != cfg.input_dim or not x.is_cuda or not xt.is_contiguous()
                or xt.dtype not in (torch.float32, torch.bfloat16)):
            raise _lib.MoEError(_lib.ERR_INVALID, "x must be the (input_dim, T) view of a contiguous float32/bfloat16 CUDA tensor")
        T = int(x.shape[1])
        if (tuple(out.shape) != (T, cfg.output_dim) or out.dtype != torch.float32 or not out.is_contiguous()
                or out.device != xt.device):
            raise _lib.MoEError(_lib.ERR_INVALID, "out must be a contiguous float32 (T, output_dim) tensor on x's device")
        if isinstance(self.balance_loss, AuxiliaryFreeLoss) and training and not self._aux_on_device:
            raise _lib.MoEError(_lib.ERR_UNSUPPORTED, "a host-side bias update needs __call__")
        if training and float(getattr(self.router, "noise_scale", 0.0) or 0.0) > 0.0:
            raise _lib.MoEError(_lib.ERR_UNSUPPORTED, "router noise is drawn per call: use __call__")
        return _BoundForward(self, xt, out, T, bool(training))

    def _forward_host(self, x, T, training, want_stats, want_routing, out=None):
        """Host buffers (NumPy arrays or torch CPU tensors, pinned or not) through
        moe_layer_forward_host: copy in, compute, copy out, synchronise."""
        cfg = self.config
        use_torch = _is_torch(x)
        if use_torch:
            import torch

            xt = x.t()
            if xt.dtype not in (torch.float32, torch.bfloat16):
                xt = xt.float()
            if not xt.is_contiguous():
                xt = xt.contiguous()
            xd = _lib.DTYPE_BF16 if xt.dtype == torch.bfloat16 else _lib.DTYPE_F32
            x_ptr = xt.data_ptr()
            if out is None:
                out = torch.empty((T, cfg.output_dim), dtype=torch.float32)
            elif (tuple(out.shape) != (T, cfg.output_dim) or out.dtype != torch.float32 or not out.is_contiguous()
                  or out.is_cuda):
                raise _lib.MoEError(_lib.ERR_INVALID, "out must be a contiguous float32 (T, output_dim) CPU tensor")
            out_ptr = out.data_ptr()
            out_view = out.t()
        else:
            if x.dtype != np.float32:
                x = x.astype(np.float32)
            xt = np.ascontiguousarray(x.T)
            xd = _lib.DTYPE_F32
            x_ptr = xt.ctypes.data
            if out is None:
                out = np.empty((T, cfg.output_dim), dtype=np.float32)
            elif out.shape != (T, cfg.output_dim) or out.dtype != np.float32 or not out.flags.c_contiguous:
                raise _lib.MoEError(_lib.ERR_INVALID, "out must be a C-ordered float32 (T, output_dim) array")
            out_ptr = out.ctypes.data
            out_view = out.T
        loss = np.zeros(1, dtype=np.float32)
        o = _lib.ForwardOutputs()
        o.loss = loss.ctypes.data
        extra = {}
        if want_stats:
            tpe = np.zeros(cfg.num_experts, dtype=np.int64)
            ent = np.zeros(1, dtype=np.float32)
            o.tokens_per_expert, o.routing_entropy = tpe.ctypes.data, ent.ctypes.data
        if want_routing:
            idx = np.empty((T, self.k_out), dtype=np.int32)
            gates = np.empty((T, self.k_out), dtype=np.float32)
            probs = np.empty((T, self.e_probs), dtype=np.float32)
            logits = np.empty((T, self.e_router), dtype=np.float32)
            o.indices, o.gates, o.probs, o.logits = idx.ctypes.data, gates.ctypes.data, probs.ctypes.data, logits.ctypes.data
            extra.update(indices=idx.T, gates=gates.T, probs=probs.T, logits=logits.T)
        _lib.check(_lib.lib.moe_layer_forward_host(self._handle, x_ptr, xd, T, int(training), out_ptr, C.byref(o)))
        if want_stats:
            extra["tokens_per_expert"] = _HostValue(tpe)
            extra["routing_entropy"] = _HostValue(ent[0])
        return out_view, np.float32(loss[0]), extra

    # -- helpers ---------------------------------------------------------------------------
    def set_profiling(self, slots: int = 1) -> None:
        """Keep per-stage CUDA events for the last ``slots`` forward calls (0 = off)."""
        _lib.check(_lib.lib.moe_layer_set_profiling(self._handle, int(slots)))

    def stage_ms(self, calls_back: int = 0) -> dict:
        """Device milliseconds per stage of the forward made ``calls_back`` calls ago."""
        ms = (C.c_float * 7)()
        _lib.check(_lib.lib.moe_layer_stage_ms(self._handle, int(calls_back), ms))
        names = ["router", "scan_loss", "permute", "gemm1", "gemm2", "combine", "exchange"]
        return dict(zip(names, [float(v) for v in ms]))

    def gemm_kernel(self, T: int) -> int:
        """0 / 1 / 2: the single-CTA, CTA-pair or two-accumulator tensor-core kernel a batch of T tokens gets."""
        n = int(_lib.lib.moe_layer_gemm_kernel(self._handle, int(T)))
        if n < 0:
            _lib.check(n)
        return n

    def tile_rows(self, T: int) -> int:
        """Rows per m-tile of the expert GEMMs for a batch of T tokens (256: CTA-pair kernel, 128:
        single-CTA tensor-core kernel, 16: FP32 kernels)."""
        n = int(_lib.lib.moe_layer_tile_rows(self._handle, int(T)))
        if n < 0:
            _lib.check(n)
        return n

    def router_rechecks(self) -> int:
        """Tokens whose logits the tensor-core router re-evaluated with FP32 FMAs since creation."""
        n = C.c_int64()
        _lib.check(_lib.lib.moe_layer_router_rechecks(self._handle, C.byref(n)))
        return int(n.value)

    def graph_replays(self) -> int:
        """Forward calls served by replaying a captured CUDA graph (small batches) since creation."""
        n = C.c_int64()
        _lib.check(_lib.lib.moe_layer_graph_replays(self._handle, C.byref(n)))
        return int(n.value)

    def launch_count(self) -> int:
        return int(_lib.lib.moe_layer_launch_count(self._handle))

    def device_status(self) -> int:
        st = C.c_int32()
        _lib.check(_lib.lib.moe_layer_device_status(self._handle, C.byref(st)))
        return st.value

    def close(self) -> None:
        if getattr(self, "_handle", None) is not None and self._handle.value:
            bl = getattr(self, "balance_loss", None)
            if getattr(self, "_aux_on_device", False) and bl._device_state is not None:
                bl._pull()                        # the loss object keeps the final state
                bl._device_state = bl._device_push = None
            _lib.lib.moe_layer_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


def create_moe_layer(input_dim: int, hidden_dim: int, output_dim: int, **kwargs) -> MoELayer:
    """create_moe_layer(input_dim, hidden_dim, output_dim; kwargs...) (src/core/moe_layer.jl:285-293).
    Keywords that MoEConfig does not know (device, compute_dtype, rng, ...) go to MoELayer."""
    cfg_fields = set(MoEConfig.__dataclass_fields__)
    cfg_kw = {k: v for k, v in kwargs.items() if k in cfg_fields}
    layer_kw = {k: v for k, v in kwargs.items() if k not in cfg_fields}
    return MoELayer(MoEConfig(input_dim=input_dim, hidden_dim=hidden_dim, output_dim=output_dim, **cfg_kw), **layer_kw)


def reset_stats(moe: MoELayer) -> None:
    """reset_stats!(moe) (src/core/moe_layer.jl:271-276)."""
    st = moe.training_stats
    st["tokens_per_expert"][:] = 0
    st["routing_entropy"].clear()
    st["capacity_overflow"] = 0


def load_balance_score(expert_counts) -> float:
    """load_balance_score(expert_counts) (src/core/utils.jl:40-52)."""
    c = np.asarray(expert_counts, dtype=np.float64)
    total = c.sum()
    if total == 0:
        return 1.0
    ideal = total / c.size
    return float(1.0 - math.sqrt(((c - ideal) ** 2).sum() / c.size) / ideal)
