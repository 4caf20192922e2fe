"""Op-layer shape arithmetic for convolutions and pooling.

Host-side mirror of tfjs-core/src/ops/conv_util.ts: computeConv2DInfo (:123-182),
computePool2DInfo (:66-86), getPadAndOutInfo (:399-435), getEffectiveFilterSize (:391-397)
and conditionalRound (:509-526).  Only the channelsLast (NHWC) layout is produced; the
backend rejects channelsFirst, as tf.fused.conv2d itself does (ops/fused_ops.ts:332-335).
"""
import math

from ._ffi import ConvInfo


def parse_tuple_param(param):
    """conv_util.ts:357-365."""
    if isinstance(param, (int, float)):
        return int(param), int(param)
    return int(param[0]), int(param[1])


def get_effective_filter_size(filter_size, dilation):
    if dilation <= 1:
        return filter_size
    return filter_size + (filter_size - 1) * (dilation - 1)


def _conditional_round(value, rounding_mode):
    if not rounding_mode:
        return value
    if rounding_mode == "round":
        return math.floor(value + 0.5)  # Math.round
    if rounding_mode == "ceil":
        return math.ceil(value)
    if rounding_mode == "floor":
        return math.floor(value)
    raise ValueError(f"Unknown roundingMode {rounding_mode}")


def _out_dim_number_pad(in_size, field, stride, pad, rounding_mode, what):
    v = _conditional_round((in_size - field + 2 * pad) / stride + 1, rounding_mode)
    if v != int(v):
        raise ValueError(f"The output # of {what} ({v}) must be an integer. "
                         "Change the stride and/or zero pad parameters")
    return int(v)


def compute_conv2d_info(in_shape, filter_shape, strides, dilations, pad, rounding_mode=None,
                        depthwise=False, data_format="channelsLast"):
    if data_format != "channelsLast":
        raise ValueError("the cuda backend supports the NHWC (channelsLast) layout only")
    batch, in_h, in_w, in_c = [int(v) for v in in_shape]
    f_h, f_w, _, f_c = [int(v) for v in filter_shape]
    s_h, s_w = parse_tuple_param(strides)
    d_h, d_w = parse_tuple_param(dilations)
    e_h = get_effective_filter_size(f_h, d_h)
    e_w = get_effective_filter_size(f_w, d_w)
    ci = ConvInfo()
    if isinstance(pad, (int, float)) and not isinstance(pad, bool):
        p = int(pad)
        top = bottom = left = right = p
        # conv_util.ts:408-414: one field size and one stride (the height's) serve both axes
        out_h = _out_dim_number_pad(in_h, e_h, s_h, p, rounding_mode, "rows")
        out_w = _out_dim_number_pad(in_w, e_h, s_h, p, rounding_mode, "columns")
    elif pad == "same":
        out_h = math.ceil(in_h / s_h)
        out_w = math.ceil(in_w / s_w)
        pad_h = max(0, (out_h - 1) * s_h + e_h - in_h)
        pad_w = max(0, (out_w - 1) * s_w + e_w - in_w)
        top = pad_h // 2
        bottom = pad_h - top
        left = pad_w // 2
        right = pad_w - left
    elif pad == "valid":
        top = bottom = left = right = 0
        out_h = math.ceil((in_h - e_h + 1) / s_h)
        out_w = math.ceil((in_w - e_w + 1) / s_w)
    else:
        raise ValueError(f"Unknown padding parameter: {pad}")
    ci.batchSize, ci.inHeight, ci.inWidth, ci.inChannels = batch, in_h, in_w, in_c
    ci.outHeight, ci.outWidth = max(out_h, 0), max(out_w, 0)
    ci.outChannels = f_c * in_c if depthwise else f_c  # conv_util.ts:151
    ci.strideHeight, ci.strideWidth = s_h, s_w
    ci.dilationHeight, ci.dilationWidth = d_h, d_w
    ci.filterHeight, ci.filterWidth = f_h, f_w
    ci.effectiveFilterHeight, ci.effectiveFilterWidth = e_h, e_w
    ci.padTop, ci.padBottom, ci.padLeft, ci.padRight = top, bottom, left, right
    return ci


def compute_pool2d_info(in_shape, filter_size, strides, dilations, pad, rounding_mode=None):
    f_h, f_w = parse_tuple_param(filter_size)
    filter_shape = [f_h, f_w, in_shape[3], in_shape[3]]
    return compute_conv2d_info(in_shape, filter_shape, strides, dilations, pad, rounding_mode, False)


def tuple_values_are_one(param):
    a, b = parse_tuple_param(param)
    return a == 1 and b == 1


def either_strides_or_dilations_are_one(strides, dilations):
    """conv_util.ts:533-536."""
    return tuple_values_are_one(strides) or tuple_values_are_one(dilations)
