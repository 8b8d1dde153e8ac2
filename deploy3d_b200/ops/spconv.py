"""``spconv_index``, ``spconv_mm``, ``bev_densify`` (deploy3d/symfun/ops/spconv/*.py)."""
import numpy as np

from ..plugins import deserialize_plugin

_CACHE = {}


def _plugin(name, data_s, cache_key=None):
    key = (name, data_s if cache_key is None else cache_key)
    plug = _CACHE.get(key)
    if plug is None:
        if len(_CACHE) > 256:
            _CACHE.clear()
        plug = _CACHE[key] = deserialize_plugin(name, data_s)
    return plug


def data_s_spconv_index(kernel_size, stride, padding, dilation, out_padding, max_num_act_out, subm, transpose):
    """Blob of SPConvIdx{N}d (deploy3d/symfun/ops/spconv/spconv_index.py:94-101; trt/spconv/index_trt.cu:39-50)."""
    data = np.array(kernel_size, dtype=np.int32).tobytes()
    data += np.array(stride, dtype=np.int32).tobytes()
    data += np.array(padding, dtype=np.int32).tobytes()
    data += np.array(dilation, dtype=np.int32).tobytes()
    data += np.array(out_padding, dtype=np.int32).tobytes()
    data += np.array([max_num_act_out], dtype=np.int32).tobytes()
    data += np.array([subm], dtype=np.bool_).tobytes()
    data += np.array([transpose], dtype=np.bool_).tobytes()
    return data


def spconv_index(in_coors, num_act_in, in_spatial_shape, kernel_size, stride, padding, dilation, out_padding,
                 max_num_act_out, subm, transpose):
    """Returns (index, num_index) when ``subm`` else (index, num_index, out_coors, num_act_out, out_spatial_shape).

    in_coors int32 [maxNumActIn, NDim+1]; num_act_in int32 [1]; in_spatial_shape: zero-element tensor
    [B, 0, D0, ..] whose *shape* carries the grid extent (deploy3d/symfun/ops/spconv/spconv_index.py:8-21)."""
    ndim = in_coors.shape[1] - 1
    data = data_s_spconv_index(kernel_size, stride, padding, dilation, out_padding, max_num_act_out, subm, transpose)
    plug = _plugin("SPConvIdx%dd" % ndim, data)
    outs = plug.enqueue(in_coors, num_act_in, in_spatial_shape)
    return outs


def data_s_spconv_mm(kernel_size, in_channels, out_channels, max_num_act_out, subm, inverse, weight, bias=None):
    """Blob of SPConvMM (deploy3d/symfun/ops/spconv/spconv_mm.py:54-63; trt/spconv/mm_trt.cu:27-37)."""
    data = np.array([int(np.prod(kernel_size))], dtype=np.int32).tobytes()
    data += np.array([in_channels], dtype=np.int32).tobytes()
    data += np.array([out_channels], dtype=np.int32).tobytes()
    data += np.array([max_num_act_out], dtype=np.int32).tobytes()
    data += np.array([subm], dtype=np.bool_).tobytes()
    data += np.array([inverse], dtype=np.bool_).tobytes()
    data += np.array([bias is not None], dtype=np.bool_).tobytes()
    data += np.ascontiguousarray(weight, dtype=np.float32).tobytes()
    if bias is not None:
        data += np.ascontiguousarray(bias, dtype=np.float32).tobytes()
    return data


def spconv_mm(in_feats, num_act_in, num_act_out, index, num_index, kernel_size, in_channels, out_channels,
              max_num_act_out, subm, inverse, weight, bias=None):
    """out_feats [maxNumActOut, Cout] in the dtype of in_feats (float16, bfloat16 or float32).

    weight: numpy [kVol, Cin, Cout] (flattened is accepted), bias: numpy [Cout] or None
    (deploy3d/symfun/ops/spconv/spconv_mm.py:21-35)."""
    data = data_s_spconv_mm(kernel_size, in_channels, out_channels, max_num_act_out, subm, inverse, weight, bias)
    plug = _plugin("SPConvMM", data)
    return plug.enqueue(in_feats, num_act_in, num_act_out, index, num_index)[0]


def data_s_bev_densify(out_channels):
    return np.array([out_channels], dtype=np.int32).tobytes()


def bev_densify(in_feats, in_coors, num_act_in, in_spatial_shape, out_channels):
    """Dense [B, C*Z, Y, X] map (deploy3d/symfun/ops/spconv/bev_densify.py:18-28)."""
    plug = _plugin("BEVDensify", data_s_bev_densify(out_channels))
    return plug.enqueue(in_feats, in_coors, num_act_in, in_spatial_shape)[0]
