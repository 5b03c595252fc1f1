"""Sparse convolution layers: SubMConv / SparseConv / SparseConvTranspose /
SparseInverseConv in 1-4 dimensions.

Constructor signatures, parameter layout (KRSC ``[C_out, *ksize, C_in]``),
initialisation, state_dict keys, ``indice_key`` reuse rules and error
messages follow the reference's spconv_triton/pytorch/conv.py; the rulebooks
and GEMMs underneath run in libspconv_b200.so.
"""

from __future__ import annotations

import math
import time as _time

import numpy as np
import torch
from torch.nn import init
from torch.nn.init import calculate_gain
from torch.nn.parameter import Parameter

from spconv_triton_b200 import SPCONV_VERSION_NUMBERS  # noqa: F401  (re-export)
from spconv_triton_b200.compat import Activation, tv
from spconv_triton_b200.constants import SAVED_WEIGHT_LAYOUT, SPCONV_DEBUG_WEIGHT
from spconv_triton_b200.core import ConvAlgo
from spconv_triton_b200.tools import nullcontext  # noqa: F401

from . import functional as Fsp
from . import ops
from ._impl import pairs as _pairs
from .core import ImplicitGemmIndiceData, IndiceData, SparseConvTensor, expand_nd, register_implicit_gemm_indice_data
from .modules import SparseModule

FILTER_HWIO = False
CPU_ONLY_BUILD = False
_NO_ACT = tv.gemm.Activation.None_
_MAX_NUM_VOXELS_DURING_TRAINING = "max_num_voxels_during_training"


class _Rulebook:
    """What one layer needs from a rulebook, whichever format it is in."""

    __slots__ = ("out_indices", "out_spatial_shape", "native", "igemm")

    def __init__(self, out_indices, out_spatial_shape, native=None, igemm=None):
        self.out_indices = out_indices
        self.out_spatial_shape = out_spatial_shape
        self.native = native  # (indice_pairs, indice_pair_num)
        self.igemm = igemm  # (pair_fwd, pair_bwd, pm_fwd, pm_bwd, ma_fwd, ma_bwd, masks)


class SparseConvolutionBase:
    def __init__(self, ndim: int, in_channels: int, out_channels: int, kernel_size=3, stride=1, padding=0,
                 dilation=1, groups: int = 1, bias: bool = True, subm: bool = False, output_padding=0,
                 transposed: bool = False, inverse: bool = False, indice_key: str | None = None,
                 algo: ConvAlgo | None = None, fp32_accum: bool | None = None,
                 record_voxel_count: bool = False, act_type: Activation = _NO_ACT, act_alpha: float = 0,
                 act_beta: float = 0, large_kernel_fast_algo: bool = False):
        if groups != 1:
            raise AssertionError("don't support groups for now")
        self.ndim = ndim
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = expand_nd(ndim, kernel_size)
        self.stride = expand_nd(ndim, stride)
        self.dilation = expand_nd(ndim, dilation)
        self.padding = expand_nd(ndim, padding)
        self.output_padding = expand_nd(ndim, output_padding)
        kv = int(np.prod(self.kernel_size))
        # a kernel volume of one is a plain matrix product; for non-subm layers
        # only when the stride is one too (k=1, s=2 still drops points)
        self.conv1x1 = kv == 1 and (subm or int(np.prod(self.stride)) == 1)
        if self.conv1x1 and not subm and self.padding != [0] * ndim:
            raise AssertionError("padding must be zero for 1x1 conv (k=1,s=1)")
        self.transposed = transposed
        self.inverse = inverse
        self.groups = groups
        self.subm = subm
        self.indice_key = indice_key
        self.record_voxel_count = record_voxel_count
        if algo is None:
            limit = 128 if large_kernel_fast_algo else 32
            algo = ConvAlgo.MaskImplicitGemm if kv <= limit else ConvAlgo.Native
        self.algo = algo
        self.fp32_accum = fp32_accum
        self.weight_shape = [out_channels, *self.kernel_size, in_channels]
        self.act_type = act_type
        self.act_alpha = act_alpha
        self.act_beta = act_beta
        if self.conv1x1 and act_type != _NO_ACT:
            raise AssertionError("conv1x1 don't support fused act")

    def is_inverseable(self):
        return self.indice_key is not None and not self.subm

    # -- forward ---------------------------------------------------------------------------

    def _output_spatial_shape(self, spatial_shape):
        if self.subm:
            return spatial_shape
        if self.transposed:
            return ops.get_deconv_output_size(spatial_shape, self.kernel_size, self.stride, self.padding,
                                              self.dilation, self.output_padding)
        return ops.get_conv_output_size(spatial_shape, self.kernel_size, self.stride, self.padding,
                                        self.dilation)

    def _open_benchmark_record(self, x, name):
        if name is None:
            raise ValueError("you need to assign name to spmodules before benchmark "
                             "(spconv.utils.bench.assign_name_to_spmod)")
        if name not in x.benchmark_record:
            x.benchmark_record[name] = {
                "type": "SparseConvolution", "indice_gen_time": [], "time": [], "num_points": [],
                "num_out_points": [],
                "params": {"kernel_size": self.kernel_size, "stride": self.stride, "padding": self.padding,
                           "dilation": self.dilation, "output_padding": self.output_padding,
                           "subm": self.subm, "transposed": self.transposed,
                           "input_channels": self.in_channels, "out_channels": self.out_channels},
            }

    def _generate(self, x, record, name, make):
        """Runs ``make()`` (a rulebook generation), timing it when benchmarking."""
        if not x.benchmark:
            return make()
        torch.cuda.synchronize()
        t0 = _time.time()
        res = make()
        torch.cuda.synchronize()
        record[name]["indice_gen_time"].append(_time.time() - t0)
        return res

    def _native_rulebook(self, x, out_tensor, indice_dict, out_spatial_shape, name) -> _Rulebook:
        datas = x.find_indice_pair(self.indice_key)
        if datas is not None and not isinstance(datas, IndiceData):
            raise AssertionError
        if self.inverse:
            if datas is None or self.indice_key is None:
                raise AssertionError
            if datas.is_subm is not False:
                raise AssertionError("inverse conv can only be used with standard conv and pool ops.")
            self._check_inverse_reuse_valid(x, x.spatial_shape, datas)
            return _Rulebook(datas.indices, datas.spatial_shape,
                             native=(datas.indice_pairs, datas.indice_pair_num))
        if self.indice_key is not None and datas is not None:
            if not self.subm:
                raise AssertionError("only support reuse subm indices")
            self._check_subm_reuse_valid(x, x.spatial_shape, datas)
            return _Rulebook(datas.out_indices, out_spatial_shape,
                             native=(datas.indice_pairs, datas.indice_pair_num))
        outids, pairs, pair_num = self._generate(
            x, out_tensor.benchmark_record, name,
            lambda: ops.get_indice_pairs(x.indices, x.batch_size, x.spatial_shape, self.algo,
                                         self.kernel_size, self.stride, self.padding, self.dilation,
                                         self.output_padding, self.subm, self.transposed))
        if self.indice_key is not None:
            if self.indice_key in indice_dict:
                raise AssertionError(f"your indice key {self.indice_key} already exists in this sparse tensor.")
            indice_dict[self.indice_key] = IndiceData(
                outids, x.indices, pairs, pair_num, x.spatial_shape, out_spatial_shape, is_subm=self.subm,
                algo=self.algo, ksize=self.kernel_size, stride=self.stride, padding=self.padding,
                dilation=self.dilation)
        return _Rulebook(outids, out_spatial_shape, native=(pairs, pair_num))

    def _igemm_rulebook(self, x, out_tensor, indice_dict, out_spatial_shape, training, name) -> _Rulebook:
        datas = x.find_indice_pair(self.indice_key)
        if datas is not None and not isinstance(datas, ImplicitGemmIndiceData):
            raise AssertionError
        if self.inverse:
            if datas is None or self.indice_key is None:
                raise AssertionError
            if datas.is_subm is not False:
                raise AssertionError("inverse conv can only be used with standard conv and pool ops.")
            self._check_inverse_reuse_valid(x, x.spatial_shape, datas)
            if x._planner is not None:
                x._planner.join_late()  # pair_bwd of the down-sampling layer may still be in the making
            # the inverse layer runs the down-sampling layer's rulebook backwards
            return _Rulebook(datas.indices, datas.spatial_shape, igemm=(
                datas.pair_bwd, datas.pair_fwd, datas.pair_mask_bwd_splits, datas.pair_mask_fwd_splits,
                datas.mask_argsort_bwd_splits, datas.mask_argsort_fwd_splits, datas.masks))
        if self.indice_key is not None and datas is not None:
            if not self.subm:
                raise AssertionError("only support reuse subm indices")
            self._check_subm_reuse_valid(x, x.spatial_shape, datas)
            return _Rulebook(datas.out_indices, out_spatial_shape, igemm=(
                datas.pair_fwd, datas.pair_bwd, datas.pair_mask_fwd_splits, datas.pair_mask_bwd_splits,
                datas.mask_argsort_fwd_splits, datas.mask_argsort_bwd_splits, datas.masks))
        planner = x._planner
        res = planner.take(self, x) if planner is not None else None
        if res is None:
            # an inference forward of a strided layer leaves the input-side tables pending
            with _pairs.deferred_backward(None if (training or self.subm) else "late"):
                res = self._generate(
                    x, out_tensor.benchmark_record, name,
                    lambda: ops.get_indice_pairs_implicit_gemm(
                        x.indices, x.batch_size, x.spatial_shape, self.algo, ksize=self.kernel_size,
                        stride=self.stride, padding=self.padding, dilation=self.dilation,
                        out_padding=self.output_padding, subm=self.subm, transpose=self.transposed,
                        is_train=(not self.subm) or training, alloc=x.thrust_allocator, timer=x._timer))
        if self.indice_key is not None:
            register_implicit_gemm_indice_data(
                indice_dict, self.indice_key, res, x.indices, is_subm=self.subm,
                spatial_shape=x.spatial_shape, out_spatial_shape=out_spatial_shape, algo=self.algo,
                ksize=self.kernel_size, stride=self.stride, dilation=self.dilation, padding=self.padding)
        return _Rulebook(res[0], out_spatial_shape, igemm=tuple(res[2:9]))

    def _conv_forward(self, training: bool, x: SparseConvTensor, weight: torch.Tensor,
                      bias: torch.Tensor | None, add_input: SparseConvTensor | None = None,
                      channel_scale: torch.Tensor | None = None, output_scale: float | None = None,
                      name: str | None = None, act_type: Activation = _NO_ACT, act_alpha: float = 0,
                      act_beta: float = 0, bn_fold=None):
        if x.is_quantized and weight.is_quantized:
            raise NotImplementedError("int8 is not supported by spconv_triton")
        if x.features.shape[1] != self.in_channels:
            raise AssertionError("channel size mismatch")
        if training and self.act_type != _NO_ACT:
            raise AssertionError("act don't support backward, only used in inference")
        # training adds the bias outside the autograd function; inference fuses it
        bias_after = bias if training else None
        bias_fused = None if training else bias
        out_spatial_shape = self._output_spatial_shape(x.spatial_shape)
        out_tensor = x.shadow_copy()
        if x.benchmark:
            self._open_benchmark_record(x, name)

        if self.conv1x1:
            # raw reinterpretation of the KRSC weight memory as [C_in, C_out], as upstream does
            feats = torch.mm(x.features, weight.view(self.in_channels, self.out_channels))
            if bias is not None:
                feats += bias
            out_tensor = out_tensor.replace_feature(feats)
            out_tensor.spatial_shape = out_spatial_shape
            return out_tensor

        indice_dict = x.indice_dict.copy()
        features = x.features.contiguous()
        if self.indice_key is not None:
            datas = x.find_indice_pair(self.indice_key)
            if datas is not None and self.algo != datas.algo:
                raise AssertionError("due to limitation of pytorch, you must provide same algo to "
                                     "layers share same indice key.")

        if self.algo == ConvAlgo.Native:
            rb = self._native_rulebook(x, out_tensor, indice_dict, out_spatial_shape, name)
        else:
            rb = self._igemm_rulebook(x, out_tensor, indice_dict, out_spatial_shape, training, name)
        n_out = rb.out_indices.shape[0]

        if x.benchmark:
            torch.cuda.synchronize()
            t_kernel = _time.time()
        if rb.native is not None:
            pairs, pair_num = rb.native
            if pairs.device != features.device:
                pairs = pairs.to(features.device)
            if self.subm:
                fn = Fsp.indice_subm_conv
            elif self.inverse:
                fn = Fsp.indice_inverse_conv
            else:
                fn = Fsp.indice_conv
            out_features = fn(features, weight, pairs, pair_num, n_out, self.algo, x._timer, bias_fused,
                              act_alpha, act_beta, act_type)
        else:
            pair_fwd, pair_bwd, pm_fwd, pm_bwd, ma_fwd, ma_bwd, masks = rb.igemm
            if training:
                # a residual input is added inside the kernel's store when nothing comes between the
                # kernel and the addition (no bias, which training adds after the kernel, no activation)
                residual = None
                if (add_input is not None and bias_after is None and self.act_type == _NO_ACT
                        and add_input.features.shape == (n_out, self.out_channels)
                        and add_input.features.device == features.device):
                    out_dt = torch.float16 if torch.is_autocast_enabled() else features.dtype
                    if add_input.features.dtype == out_dt:
                        residual, add_input = add_input.features, None
                out_features = Fsp.implicit_gemm(features, weight, pair_fwd, pair_bwd, pm_fwd, pm_bwd, ma_fwd,
                                                 ma_bwd, n_out, masks, training, self.subm, x._timer,
                                                 self.fp32_accum, bias_fused, act_alpha, act_beta, act_type,
                                                 residual)
            else:
                out_features, _, _ = ops.implicit_gemm(
                    features, weight, pair_fwd, pm_fwd, ma_fwd, n_out, masks, training, self.subm, x._timer,
                    self.fp32_accum, bias_fused, act_alpha, act_beta, act_type,
                    1.0 if output_scale is None else output_scale, channel_scale,
                    output_add=add_input.features if add_input is not None else None, output_add_scale=0.0,
                    output_dtype=weight.dtype if output_scale is None else None, _bn_fold=bn_fold)
        if bias_after is not None:
            out_features += bias_after
        if x.benchmark:
            torch.cuda.synchronize()
            rec = out_tensor.benchmark_record[name]
            rec["time"].append(_time.time() - t_kernel)
            rec["num_points"].append(features.shape[0])
            rec["num_out_points"].append(out_features.shape[0])
        if (not self.subm and not self.inverse and self.record_voxel_count
                and hasattr(self, _MAX_NUM_VOXELS_DURING_TRAINING)):
            ops.maximum_value_int_(getattr(self, _MAX_NUM_VOXELS_DURING_TRAINING), n_out)

        out_tensor = out_tensor.replace_feature(out_features)
        out_tensor.indices = rb.out_indices
        out_tensor.indice_dict = indice_dict
        out_tensor.spatial_shape = rb.out_spatial_shape
        if add_input is not None:
            out_tensor = out_tensor.replace_feature(ops._apply_act_inplace(
                out_tensor.features + add_input.features, self.act_type, self.act_alpha, self.act_beta))
        return out_tensor

    # -- reuse checks ------------------------------------------------------------------------

    def _check_subm_reuse_valid(self, inp: SparseConvTensor, spatial_shape, datas):
        if not datas.is_subm:
            raise AssertionError("only support reuse subm indices")
        if self.kernel_size != datas.ksize:
            raise ValueError(f"subm with same indice_key must have same kernel size, expect {datas.ksize}, "
                             f"this layer {self.kernel_size}")
        if self.dilation != datas.dilation:
            raise ValueError(f"subm with same indice_key must have same dilation, expect {datas.dilation}, "
                             f"this layer {self.dilation}")
        if inp.spatial_shape != datas.spatial_shape:
            raise ValueError(f"subm with same indice_key must have same spatial structure, expect "
                             f"{datas.spatial_shape}, input {spatial_shape}")
        if inp.indices.shape[0] != datas.indices.shape[0]:
            raise ValueError(f"subm with same indice_key must have same num of indices, expect "
                             f"{datas.indices.shape[0]}, input {inp.indices.shape[0]}")

    def _check_inverse_reuse_valid(self, inp: SparseConvTensor, spatial_shape, datas):
        if self.kernel_size != datas.ksize:
            raise ValueError(f"Inverse with same indice_key must have same kernel size, expect {datas.ksize}, "
                             f"this layer {self.kernel_size}, please check Inverse Convolution in docs/USAGE.md.")
        if inp.spatial_shape != datas.out_spatial_shape:
            raise ValueError(f"Inverse with same indice_key must have same spatial structure (spatial shape), "
                             f"expect {datas.spatial_shape}, input {spatial_shape}, "
                             "please check Inverse Convolution in docs/USAGE.md.")
        if inp.indices.shape[0] != datas.out_indices.shape[0]:
            raise ValueError(f"Inverse with same indice_key must have same num of indices, expect "
                             f"{datas.indices.shape[0]}, input {inp.indices.shape[0]}, "
                             "please check Inverse Convolution in .")


class SparseConvolution(SparseConvolutionBase, SparseModule):
    __constants__ = ["stride", "padding", "dilation", "groups", "bias", "subm", "inverse", "transposed",
                     "output_padding"]

    def __init__(self, ndim: int, in_channels: int, out_channels: int, kernel_size=3, stride=1, padding=0,
                 dilation=1, groups: int = 1, bias: bool = True, subm: bool = False, output_padding=0,
                 transposed: bool = False, inverse: bool = False, indice_key: str | None = None,
                 algo: ConvAlgo | None = None, fp32_accum: bool | None = None,
                 record_voxel_count: bool = False, act_type: Activation = _NO_ACT, act_alpha: float = 0,
                 act_beta: float = 0, large_kernel_fast_algo: bool = False, name=None, device=None,
                 dtype=None):
        SparseConvolutionBase.__init__(
            self, ndim, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias=False,
            subm=subm, output_padding=output_padding, transposed=transposed, inverse=inverse,
            indice_key=indice_key, algo=algo, fp32_accum=fp32_accum, record_voxel_count=record_voxel_count,
            act_type=act_type, act_alpha=act_alpha, act_beta=act_beta,
            large_kernel_fast_algo=large_kernel_fast_algo)
        SparseModule.__init__(self, name=name)
        if record_voxel_count and not self.subm and not self.inverse:
            self.register_buffer(_MAX_NUM_VOXELS_DURING_TRAINING,
                                 torch.zeros(1, dtype=torch.int32, device=device))
        self.weight = Parameter(torch.zeros(*self.weight_shape, device=device, dtype=dtype))
        if bias:
            self.bias = Parameter(torch.zeros(out_channels, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        self._register_load_state_dict_pre_hook(self._load_weight_different_layout)

    def get_max_num_voxels(self) -> torch.Tensor | None:
        return getattr(self, _MAX_NUM_VOXELS_DURING_TRAINING, None)

    def _load_weight_different_layout(self, state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs):
        counter = prefix + _MAX_NUM_VOXELS_DURING_TRAINING
        if self.record_voxel_count and not self.subm and not self.inverse and counter not in state_dict:
            state_dict[counter] = torch.zeros(1, dtype=torch.int32)
        if not SAVED_WEIGHT_LAYOUT or SAVED_WEIGHT_LAYOUT == "KRSC":
            return
        key = prefix + "weight"
        if key not in state_dict:
            raise AssertionError
        nd = self.ndim
        perm = {"RSKC": (nd, *range(nd), nd + 1), "RSCK": (nd + 1, *range(nd), nd)}[SAVED_WEIGHT_LAYOUT]
        # Upstream applies the permutation twice, so a checkpoint stored in a
        # non-KRSC layout ends with a shape mismatch; kept for identical behaviour.
        for _ in range(2):
            state_dict[key] = state_dict[key].permute(*perm).contiguous()

    def extra_repr(self):
        parts = [f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}"]
        if self.padding != (0,) * len(self.padding):
            parts.append(f"padding={self.padding}")
        if self.dilation != (1,) * len(self.dilation):
            parts.append(f"dilation={self.dilation}")
        if self.output_padding != (0,) * len(self.output_padding):
            parts.append(f"output_padding={self.output_padding}")
        if self.groups != 1:
            parts.append(f"groups={self.groups}")
        if self.bias is None:
            parts.append("bias=False")
        if self.algo is not None:
            parts.append(f"algo={self.algo}")
        if self.act_type != _NO_ACT:
            parts.append(f"act={self.act_type}")
        return ", ".join(parts)

    def _calculate_fan_in_and_fan_out(self):
        rf = int(np.prod(self.kernel_size))
        return self.in_channels * rf, self.out_channels * rf

    def _calculate_correct_fan(self, mode):
        mode = mode.lower()
        if mode not in ("fan_in", "fan_out"):
            raise ValueError(f"Mode {mode} not supported, please use one of ['fan_in', 'fan_out']")
        fan_in, fan_out = self._calculate_fan_in_and_fan_out()
        return fan_in if mode == "fan_in" else fan_out

    def _custom_kaiming_uniform_(self, tensor, a=0, mode="fan_in", nonlinearity="leaky_relu"):
        """kaiming_uniform_ with the fan computed for the KRSC layout."""
        bound = math.sqrt(3.0) * calculate_gain(nonlinearity, a) / math.sqrt(self._calculate_correct_fan(mode))
        with torch.no_grad():
            return tensor.uniform_(-bound, bound)

    def reset_parameters(self):
        self._custom_kaiming_uniform_(self.weight, a=math.sqrt(0.005 if SPCONV_DEBUG_WEIGHT else 5))
        if self.bias is not None:
            fan_in, _ = self._calculate_fan_in_and_fan_out()
            bound = 1 / math.sqrt(fan_in)
            init.uniform_(self.bias, -bound, bound)

    # data-dependent shapes and raw CUDA launches: keep torch.compile out of here
    def can_fold_epilogue(self) -> bool:
        """True if an inference BatchNorm (and ReLU) that follows this layer can be
        applied inside its GEMM kernel: evaluation mode, implicit-gemm algorithm,
        a real convolution (not the 1x1 matrix-product shortcut), no activation of
        its own."""
        return (not self.training and not self.conv1x1 and self.algo != ConvAlgo.Native
                and self.act_type == _NO_ACT)

    @torch.compiler.disable
    def forward(self, x: SparseConvTensor, add_input: SparseConvTensor | None = None, _fold=None):
        """``_fold = (scale, shift, relu)`` is used by SparseSequential to hand the
        layer a folded BatchNorm + ReLU (see modules.py)."""
        act_type, bn_fold = self.act_type, None
        if _fold is not None:
            scale, shift, relu = _fold
            bn_fold = (scale, shift)
            if relu:
                act_type = tv.gemm.Activation.ReLU
        return self._conv_forward(self.training, x, self.weight, self.bias, add_input, name=self.name,
                                  act_type=act_type, act_alpha=self.act_alpha, act_beta=self.act_beta,
                                  bn_fold=bn_fold)


def _leaf(name: str, ndim: int, flavour: str):
    """Builds one of the 16 public layer classes.  ``flavour`` selects the
    constructor signature of the family (regular / transpose / inverse / subm)."""
    if flavour in ("conv", "transpose"):
        transposed = flavour == "transpose"

        class Leaf(SparseConvolution):
            def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1,
                         groups=1, bias=True, indice_key=None, algo: ConvAlgo | None = None,
                         fp32_accum: bool | None = None, record_voxel_count: bool = False,
                         large_kernel_fast_algo: bool = False, name=None):
                super().__init__(ndim, in_channels, out_channels, kernel_size, stride, padding, dilation,
                                 groups, bias, transposed=transposed, indice_key=indice_key, algo=algo,
                                 fp32_accum=fp32_accum, record_voxel_count=record_voxel_count,
                                 large_kernel_fast_algo=large_kernel_fast_algo, name=name)
    elif flavour == "inverse":

        class Leaf(SparseConvolution):
            def __init__(self, in_channels, out_channels, kernel_size, indice_key, bias=True,
                         algo: ConvAlgo | None = None, fp32_accum: bool | None = None,
                         large_kernel_fast_algo: bool = False, name=None):
                super().__init__(ndim, in_channels, out_channels, kernel_size, bias=bias, inverse=True,
                                 indice_key=indice_key, algo=algo, fp32_accum=fp32_accum,
                                 large_kernel_fast_algo=large_kernel_fast_algo, name=name)
    else:

        class Leaf(SparseConvolution):
            def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1,
                         groups=1, bias=True, indice_key=None, algo: ConvAlgo | None = None,
                         fp32_accum: bool | None = None, large_kernel_fast_algo: bool = False, name=None):
                super().__init__(ndim, in_channels, out_channels, kernel_size, stride, padding, dilation,
                                 groups, bias, True, indice_key=indice_key, algo=algo, fp32_accum=fp32_accum,
                                 large_kernel_fast_algo=large_kernel_fast_algo, name=name)

    Leaf.__name__ = Leaf.__qualname__ = name
    Leaf.__module__ = __name__
    return Leaf


for _nd in (1, 2, 3, 4):
    for _prefix, _flavour in (("SparseConv", "conv"), ("SparseConvTranspose", "transpose"),
                              ("SparseInverseConv", "inverse"), ("SubMConv", "subm")):
        _cls_name = f"{_prefix}{_nd}d"
        globals()[_cls_name] = _leaf(_cls_name, _nd, _flavour)
del _nd, _prefix, _flavour, _cls_name

DEFAULT_SPARSE_CONV_TYPES = {globals()[f"{p}{d}d"] for p in ("SubMConv", "SparseConv", "SparseInverseConv",
                                                              "SparseConvTranspose") for d in (1, 2, 3, 4)}

__all__ = ["SparseConvolution", "SparseConvolutionBase"] + [
    f"{p}{d}d" for p in ("SparseConv", "SparseConvTranspose", "SparseInverseConv", "SubMConv") for d in (1, 2, 3, 4)]
