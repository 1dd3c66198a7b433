"""Linear / matmul layers over the B200 binary GEMM, with the class names and call signatures of the
reference's ``tests/python/bgemm_linear.py`` so that its users can switch imports unchanged.

Forward passes run on the GPU through the ``lowbit_kernel`` extension (sm_100a kernels; there is no CPU
or eager fallback for them). Backward passes keep the reference's straight-through formulas and run as
ordinary torch ops: they are dense floating-point GEMMs, not part of the 1-bit hot path.

What differs from the reference, on purpose:
  * no ``x.shape[0] % 32`` / ``K % 128`` / ``M % 32`` restrictions (bgemm_linear.py:475,505,555,586);
  * inputs with more than two dimensions are flattened over their leading dimensions for the forward;
  * ``NNLinear_elastic_signed`` (binary weight x ternary activation, pure torch in the reference,
    bgemm_linear.py:246-275) runs on the GPU kernel as well;
  * ``BinaryLinear`` / ``BinaryMLP`` / ``bgemm_attn_matmul_batched`` are additions: prepacked weights,
    fused per-channel scale, batched heads.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

import lowbit_kernel

__all__ = [
    "BNNLinear", "BGEMMLinear", "BGEMMLinear_elastic_signed", "bgemm_matmul", "bgemm_attn_matmul",
    "BGEMMLinear_bireal", "NNLinear_elastic_signed", "BinaryLinear", "BinaryMLP", "bgemm_attn_matmul_batched",
]

AND_POP, XOR_POP, ATTN_MM, BWTA = 0, 1, 2, 3
_ACT_SIGN, _ACT_TERNARY = 0, 1
_WBIT_NONZERO, _WBIT_NEGATIVE_NZ = 2, 3
_OUT_I32, _OUT_F16, _OUT_F16_SCALED = 0, 1, 2


def _instr(instruction: str) -> int:
    return AND_POP if instruction == "and" else XOR_POP          # 'xor' is the default, as in the reference


def _kernel_2d(x: torch.Tensor, w: torch.Tensor, instr: int) -> torch.Tensor:
    """[*, K] x [M, K] -> [*, M] fp16 through the drop-in extension call."""
    lead = x.shape[:-1]
    out = lowbit_kernel.bgemm_linear_forward_cuda(x.reshape(-1, x.shape[-1]), w, 1, instr)
    return out.reshape(*lead, w.shape[0])


def _ste_grads(x_sign: torch.Tensor, w_sign: torch.Tensor, grad_output: torch.Tensor):
    """d(x @ w.T)/dx and /dw for 2-D or batched 3-D activations with a shared 2-D weight."""
    if w_sign.dim() != 2:
        raise AssertionError("weight dim must be 2, now is %d" % w_sign.dim())
    if x_sign.dim() == 3:
        w_grad = torch.bmm(x_sign.transpose(1, 2), grad_output).transpose(1, 2)
        x_grad = torch.bmm(grad_output, w_sign.repeat(x_sign.shape[0], 1, 1))
    else:
        x_grad = torch.mm(grad_output, w_sign)
        w_grad = torch.mm(x_sign.T, grad_output).T
    return x_grad, w_grad


# --------------------------------------------------------------------------------------------------
# autograd functions (reference: bgemm_linear.py:9-219)
# --------------------------------------------------------------------------------------------------
class bgemm_matmul(torch.autograd.Function):
    """{-1,+1} x {-1,+1} (or {0,1} with instruction='and') product matA @ matB, both binarised by sign.

    Backward is the straight-through gradient of A @ B. (The reference's formulas, bgemm_linear.py:28-42, multiply
    grad_output by matB without transposing it, which only has consistent shapes when matB is square.)
    """

    @staticmethod
    def forward(ctx, matA, matB, instruction="xor"):
        matA, matB = matA.to(torch.half), matB.to(torch.half)
        ctx.save_for_backward(matA, matB)
        return _kernel_2d(matA, matB.transpose(-1, -2), _instr(instruction))

    @staticmethod
    def backward(ctx, grad_output):
        matA, matB = ctx.saved_tensors
        a, b = matA.sign(), matB.sign()
        if b.dim() != 2:
            raise AssertionError("matB dim must be 2, now is %d" % b.dim())
        if a.dim() == 3:
            b_grad = torch.bmm(a.transpose(1, 2), grad_output).sum(dim=0)
            a_grad = torch.matmul(grad_output, b.T)
        else:
            b_grad = torch.mm(a.T, grad_output)
            a_grad = torch.mm(grad_output, b.T)
        return a_grad, b_grad, None


class bgemm_attn_matmul(torch.autograd.Function):
    """attn @ value with attn read as a {0,1} mask ("1" where the sign bit is clear) and value as {-1,+1}."""

    @staticmethod
    def forward(ctx, input1, input2, instruction="attn_mm"):
        input1, input2 = input1.to(torch.half), input2.to(torch.half)
        ctx.save_for_backward(input1, input2)
        if input1.dim() == 3:
            return lowbit_kernel.bgemm_attn_matmul_batched(input1, input2, False)
        return lowbit_kernel.bgemm_linear_forward_cuda(input2.transpose(-1, -2).contiguous(), input1, 1, ATTN_MM).T

    @staticmethod
    def backward(ctx, grad_output):
        input1, input2 = ctx.saved_tensors
        mask = (input1.sign() + 1) / 2
        mask = torch.where(mask == 0, torch.ones_like(mask), mask)
        val = input2.sign()
        if mask.dim() != 2:
            raise AssertionError("input1 dim must be 2, now is %d" % mask.dim())
        if val.dim() == 3:
            g1 = torch.bmm(grad_output, val.T).transpose(1, 2) / 2
            g2 = torch.bmm(mask.transpose(1, 2).repeat(val.shape[0], 1, 1), grad_output)
        else:
            g1 = torch.mm(grad_output, val.T) / 2
            g2 = torch.mm(mask.T, grad_output)
        return g1, g2, None


class bgemm_linear(torch.autograd.Function):
    """sign(input) @ sign(weight).T with a straight-through backward."""

    @staticmethod
    def forward(ctx, input, weight, instruction="xor"):
        input, weight = input.to(torch.half), weight.to(torch.half)
        ctx.save_for_backward(input, weight)
        return _kernel_2d(input, weight, _instr(instruction))

    @staticmethod
    def backward(ctx, grad_output):
        x, w = ctx.saved_tensors
        x_grad, w_grad = _ste_grads(x.sign(), w.sign(), grad_output)
        return x_grad, w_grad, None


class bgemm_linear_bireal(torch.autograd.Function):
    """Same forward; the activation gradient is shaped by the Bi-Real triangle 2 - 2|x| on |x| <= 1."""

    @staticmethod
    def forward(ctx, input, weight, instruction="xor"):
        input, weight = input.to(torch.half), weight.to(torch.half)
        ctx.save_for_backward(input, weight)
        return _kernel_2d(input, weight, _instr(instruction))

    @staticmethod
    def backward(ctx, grad_output):
        x, w = ctx.saved_tensors
        x_grad, w_grad = _ste_grads(x.sign(), w.sign(), grad_output)
        ax = x.abs()
        ax = torch.where(ax > 1, torch.ones_like(ax), ax)
        return x_grad * (2 - 2 * ax), w_grad, None


def ternary(x, is_act):
    """{-1, 0, +1} by torch.sign (bgemm_linear.py:222-241)."""
    return x.sign()


def calculate_gradient_signed(qx, grad, grad_scale, is_act=True):
    """Gradient w.r.t. the quantisation scale of an elastic signed quantiser with range [-1, 1]."""
    lo, hi = -1, 1
    small = (qx < lo).float()
    big = (qx > hi).float()
    middle = 1.0 - small - big
    if is_act:
        grad_s = ((small * lo + big * hi + middle * (ternary(qx, is_act) - qx)) * grad * grad_scale).sum(dim=-1).unsqueeze(dim=0)
    else:
        grad_s = (ternary(qx, is_act) * grad * grad_scale).sum(dim=-1).unsqueeze(dim=0)
    return grad, grad_s


def _elastic_backward(ctx, grad_output, clip, shape_fn, weight_is_act):
    x, w = ctx.saved_tensors
    grad_scale = ctx.other
    x_grad, w_grad = _ste_grads(ternary(x, True), ternary(w, False), grad_output)
    gx, g_sa = calculate_gradient_signed(x, x_grad, grad_scale, True)
    _, g_sw = calculate_gradient_signed(w, w_grad, grad_scale, weight_is_act)
    ax = x.abs()
    ax = torch.where(ax > clip, torch.ones_like(ax) * clip, ax)
    gx = gx * shape_fn(ax)
    aw = w.abs()
    aw = torch.where(aw > clip, torch.ones_like(aw) * clip, aw)
    w_grad = w_grad * shape_fn(aw)
    return gx, w_grad, g_sa, g_sw, None


def _center_and_scale(input, weight, sa):
    x = input.clone()
    w = weight.clone()
    x -= x.mean().item()
    w -= w.mean().item()
    return x / sa, w


class nn_linear_elastic_signed(torch.autograd.Function):
    """Binary/ternary weight x ternary activation (BWTA): ternary(x/sa) @ ternary(w).T * sa * sw.

    The reference evaluates the product with a dense torch matmul (bgemm_linear.py:246-275); here it is
    two 1-bit GEMMs on the GPU -- a sign plane and a non-zero plane of the weights against int8 ternary
    activations -- so that weights that are exactly zero contribute 0 as torch.sign makes them.
    """

    @staticmethod
    def forward(ctx, input, weight, sa, sw, grad_scale, instruction="xor"):
        x, w = _center_and_scale(input, weight, sa)
        ctx.other = grad_scale
        ctx.save_for_backward(x, w)
        xh, wh = x.to(torch.half), w.to(torch.half)
        lead = xh.shape[:-1]
        x2 = xh.reshape(-1, xh.shape[-1])
        M, K = wh.shape
        acts, colsum = lowbit_kernel.prepare_acts(x2, _ACT_TERNARY, False)
        neg_plane = lowbit_kernel.binary_weight_prepacking_cuda(wh, _WBIT_NEGATIVE_NZ)
        nz_plane = lowbit_kernel.binary_weight_prepacking_cuda(wh, _WBIT_NONZERO)
        d_neg = lowbit_kernel.gemm_prepared(neg_plane, M, K, acts, colsum, AND_POP, _OUT_I32, 0, None, 0)
        d_nz = lowbit_kernel.gemm_prepared(nz_plane, M, K, acts, colsum, AND_POP, _OUT_I32, 0, None, 0)
        out = (d_nz - 2 * d_neg).to(xh.dtype).reshape(*lead, M)
        return out * sa * sw

    @staticmethod
    def backward(ctx, grad_output):
        return _elastic_backward(ctx, grad_output, 1, lambda t: 2 * torch.exp(-t ** 2), False)


class bgemm_linear_elastic_signed(torch.autograd.Function):
    """sign(x/sa) @ sign(w).T * sa * sw after removing the scalar means (bgemm_linear.py:350-380)."""

    @staticmethod
    def forward(ctx, input, weight, sa, sw, grad_scale, instruction="xor"):
        x, w = _center_and_scale(input, weight, sa)
        ctx.other = grad_scale
        ctx.save_for_backward(x, w)
        out = _kernel_2d(x.to(torch.half), w.to(torch.half), _instr(instruction))
        return out * sa * sw

    @staticmethod
    def backward(ctx, grad_output):
        x, w = ctx.saved_tensors
        grad_scale = ctx.other
        x_grad, w_grad = _ste_grads(x.sign(), w.sign(), grad_output)
        gx, g_sa = calculate_gradient_signed(x, x_grad, grad_scale, True)
        _, g_sw = calculate_gradient_signed(w, w_grad, grad_scale, True)
        clip = 4
        shape_fn = lambda t: 2 / torch.cosh(t) ** 2          # noqa: E731
        ax = x.abs()
        ax = torch.where(ax > clip, torch.ones_like(ax) * clip, ax)
        aw = w.abs()
        aw = torch.where(aw > clip, torch.ones_like(aw) * clip, aw)
        return gx * shape_fn(ax), w_grad * shape_fn(aw), g_sa, g_sw, None


# --------------------------------------------------------------------------------------------------
# modules (reference: bgemm_linear.py:460-645)
# --------------------------------------------------------------------------------------------------
class _LazyScaledLinear(nn.Linear):
    """nn.Linear whose quantisation scales are initialised from the first batch it sees."""

    def __init__(self, in_channels, out_channels, bias=False):
        super().__init__(in_channels, out_channels, bias)
        self.initialized = False

    def _initialize(self, x, w):
        assert not self.initialized, "already initialized."
        self.sw = nn.Parameter(w.norm(1, 1).div(w.nelement()), requires_grad=True)      # per-row L1 / total count
        self.sa = nn.Parameter(2 * x.abs().mean(), requires_grad=True)
        self.grad_scale = 1.0 / math.sqrt(x.numel())
        self.zpw = torch.mean(w).detach()
        self.zpa = torch.mean(x).detach()
        self.initialized = True

    def _add_bias(self, out):
        if self.bias is not None:
            out += self.bias.view(1, -1).expand_as(out)
        return out

    def _inference(self, x) -> bool:
        """No gradient will be asked for: the packed weight plane can be kept between calls."""
        return not (torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad))

    def _cached_plane(self):
        """Packed sign plane of (weight - zpw), re-packed only when the weight has been written since (its version
        counter) or replaced. The reference packs the fp16 weight inside the kernel on every call."""
        key = (self.weight._version, self.weight.data_ptr(), self.weight.device)
        if getattr(self, "_plane_key", None) != key:
            w = (self.weight.detach() - self.zpw).to(torch.half)
            self._plane = lowbit_kernel.binary_weight_prepacking_cuda(w, 0)
            self._plane_key = key
        return self._plane

    def _forward_cached(self, x):
        """sign(x - zpa) @ sign(weight - zpw).T through the prepacked plane: the same bits as the drop-in call."""
        lead, K, M = x.shape[:-1], self.in_features, self.out_features
        x2 = (x - self.zpa).to(torch.half).reshape(-1, K)
        out = lowbit_kernel.bgemm_linear_forward_packed(x2, self._cached_plane(), M, K, None, 0, XOR_POP, _OUT_F16)
        return out.reshape(*lead, M)


class BGEMMLinear(_LazyScaledLinear):
    def forward(self, x):
        if not self.initialized:
            self._initialize(x, self.weight)
        if self._inference(x):
            return self._add_bias(self._forward_cached(x) * self.sw * self.sa)
        out = bgemm_linear.apply(x - self.zpa, self.weight - self.zpw) * self.sw * self.sa
        return self._add_bias(out)


class BGEMMLinear_bireal(_LazyScaledLinear):
    def forward(self, x):
        if not self.initialized:
            self._initialize(x, self.weight)
        if self._inference(x):
            return self._add_bias(self._forward_cached(x) * self.sw * self.sa)
        out = bgemm_linear_bireal.apply(x - self.zpa, self.weight - self.zpw) * self.sw * self.sa
        return self._add_bias(out)


class BGEMMLinear_elastic_signed(_LazyScaledLinear):
    def __init__(self, in_channels, out_channels, bias=True):
        super().__init__(in_channels, out_channels, bias)

    def forward(self, x):
        if not self.initialized:
            self._initialize(x, self.weight)
        out = bgemm_linear_elastic_signed.apply(x, self.weight, self.sa, self.sw, self.grad_scale)
        return self._add_bias(out)


class NNLinear_elastic_signed(_LazyScaledLinear):
    def __init__(self, in_channels, out_channels, bias=True):
        super().__init__(in_channels, out_channels, bias)

    def forward(self, x):
        if not self.initialized:
            self._initialize(x, self.weight)
        out = nn_linear_elastic_signed.apply(x, self.weight, self.sa, self.sw, self.grad_scale)
        return self._add_bias(out)


class BinActive(torch.autograd.Function):
    """sign with sign(0) = +1; identity gradient."""

    @staticmethod
    def forward(ctx, input):
        s = input.sign()
        return torch.where(s == 0, torch.ones_like(s), s)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output.clone()


class BNNLinear(_LazyScaledLinear):
    """Dense torch twin of BGEMMLinear (bgemm_linear.py:619-645): the numerical reference of the binary layers."""

    def forward(self, x):
        if not self.initialized:
            self._initialize(x, self.weight)
        bw = BinActive.apply(self.weight - self.zpw)
        bx = BinActive.apply(x - self.zpa)
        return nn.functional.linear(bx, bw, self.bias) * self.sw * self.sa


# --------------------------------------------------------------------------------------------------
# additions: prepacked inference layers and the batched attention product
# --------------------------------------------------------------------------------------------------
def bgemm_attn_matmul_batched(attn: torch.Tensor, value: torch.Tensor, exact: bool = False) -> torch.Tensor:
    """[B, Sq, Sk] {0,1}-mask ("1" = sign bit clear) @ [B, Sk, d] {-1,+1} -> [B, Sq, d] in ONE launch sequence."""
    return lowbit_kernel.bgemm_attn_matmul_batched(attn, value, exact)


class BinaryLinear(nn.Module):
    """Inference layer with weights sign-binarised once: y = alpha * (sign(w) @ act(x)), fp16 out.

    alpha[m] = mean |w[m, :]| (per output channel). Activations are binarised by sign (+0 -> +1) or, with
    ternary=True, by torch.sign. The scale is applied inside the GEMM epilogue.

    The layer's only buffer is `packed`: the packed-weight bundle (header with magic and layout version, tiled
    bit plane, row bit counts, scales), so `state_dict()` round trips carry their own layout description and a
    bundle written by another layout version is refused when it is loaded. `plane` and `alpha` are views into it.
    """

    def __init__(self, weight: torch.Tensor, ternary: bool = False, alpha: torch.Tensor | None = None):
        super().__init__()
        assert weight.is_cuda and weight.dim() == 2
        self.out_features, self.in_features = weight.shape
        self.register_buffer("packed", lowbit_kernel.binary_weight_prepacking_bundle_cuda(weight, 0))
        # The weights never change after this point: once the prepack has finished, forward calls may promise the
        # kernels "static weights" (they then fetch weights while the previous kernel of the stream still runs).
        torch.cuda.current_stream(weight.device).synchronize()
        self.ternary = ternary
        self._views = None
        if alpha is not None:
            self.alpha.copy_(alpha.to(torch.half).to(weight.device))

    def _open(self):
        key = (self.packed.data_ptr(), self.packed.numel())
        if self._views is None or self._views[0] != key:
            plane, alpha, rowpop, M, K, wbit = lowbit_kernel.unpack_bundle(self.packed)       # validates magic / version / sizes
            if (M, K) != (self.out_features, self.in_features) or wbit != 0:
                raise RuntimeError(f"packed weights describe a {M} x {K} matrix (bit mode {wbit}), the layer is "
                                   f"{self.out_features} x {self.in_features}")
            self._views = (key, plane, alpha, rowpop)
        return self._views

    @property
    def plane(self) -> torch.Tensor:
        return self._open()[1]

    @property
    def alpha(self) -> torch.Tensor:
        return self._open()[2]

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self._views = None
        self._open()                      # a bundle of another layout version or shape fails here, not in a kernel

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        out = lowbit_kernel.bgemm_linear_forward_packed(
            x.reshape(-1, self.in_features), self.plane, self.out_features, self.in_features, self.alpha, 0,
            BWTA if self.ternary else XOR_POP, _OUT_F16_SCALED, True)
        return out.reshape(*lead, self.out_features)

    @property
    def op(self) -> int:
        return BWTA if self.ternary else XOR_POP

    @property
    def act_mode(self) -> int:
        return _ACT_TERNARY if self.ternary else _ACT_SIGN

    def prepare(self, x: torch.Tensor):
        """fp16 [N, in_features] -> this layer's prepared activations (int8 rows, row sums)."""
        return lowbit_kernel.prepare_acts(x.reshape(-1, self.in_features), self.act_mode, False)

    def forward_prepared(self, acts: torch.Tensor, colsum: torch.Tensor, next_layer: "BinaryLinear | None" = None, sums: "torch.Tensor | None" = None):
        """GEMM on prepared activations. With next_layer the scaled result is turned into that layer's prepared
        activations inside the GEMM epilogue (no fp16 round trip) and (acts, colsum) is returned; else fp16 [N, out].
        `sums`: an int32 tensor, zeroed by the caller on the current stream, that receives the new row sums (the call
        then enqueues nothing but its kernel)."""
        if next_layer is None:
            return lowbit_kernel.gemm_prepared(self.plane, self.out_features, self.in_features, acts, colsum, self.op, _OUT_F16_SCALED, 0,
                                               self.alpha, 0, True)
        assert next_layer.in_features == self.out_features
        return lowbit_kernel.gemm_prepared_to_acts(self.plane, self.out_features, self.in_features, acts, colsum, self.op,
                                                   next_layer.act_mode, self.alpha, 0, sums)


class BinaryMLP(nn.Module):
    """Stack of BinaryLinear layers; the sign of each fp16 output is the next layer's binary input.

    fused=True (default) keeps activations on the int8 path between layers: one activation pass for the input,
    then one GEMM per layer whose epilogue writes the next layer's activations (same bits as the unfused chain).
    graph=True replays the whole forward from a CUDA graph captured per input shape:
    a small MLP is bound by launch latency, not by the kernels. The input is copied into the graph's static
    buffer and the result is returned as a copy.
    """

    def __init__(self, weights, graph: bool = False, fused: bool = True):
        super().__init__()
        self.layers = nn.ModuleList(BinaryLinear(w) for w in weights)
        self.graph = graph
        self.fused = fused      # hidden layers produce the next layer's int8 activations in their GEMM epilogue
        self._captured = {}

    def _eager(self, x: torch.Tensor) -> torch.Tensor:
        if not self.fused:
            for layer in self.layers:
                x = layer(x)
            return x
        # one activation pass for the input, then every hidden layer hands int8 activations to the next one
        lead = x.shape[:-1]
        # Under stream capture the row sums of all hidden layers' activations live in one array, zeroed by one fill ahead of
        # the chain: nothing but kernels stands between the GEMMs of the graph (a memset node there costs ~4 us per layer).
        # Eager calls are bound by host time, and the library's own memset per layer is the cheaper call there.
        sums = None
        if len(self.layers) > 1 and torch.cuda.is_current_stream_capturing():
            sums = torch.zeros((len(self.layers) - 1, x.numel() // x.shape[-1]), dtype=torch.int32, device=x.device)
        acts, colsum = self.layers[0].prepare(x)
        for i, layer in enumerate(self.layers[:-1]):
            acts, colsum = layer.forward_prepared(acts, colsum, self.layers[i + 1], None if sums is None else sums[i])
        y = self.layers[-1].forward_prepared(acts, colsum)
        return y.reshape(*lead, self.layers[-1].out_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.graph:
            return self._eager(x)
        key = (tuple(x.shape), x.dtype, x.device)
        entry = self._captured.get(key)
        if entry is None:
            static_x = x.clone()
            side = torch.cuda.Stream(device=x.device)
            side.wait_stream(torch.cuda.current_stream(x.device))
            with torch.cuda.stream(side):          # first calls set kernel attributes and size the workspaces
                for _ in range(2):
                    self._eager(static_x)
            torch.cuda.current_stream(x.device).wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                static_y = self._eager(static_x)
            entry = self._captured[key] = (g, static_x, static_y)
        g, static_x, static_y = entry
        static_x.copy_(x)
        g.replay()
        return static_y.clone()
