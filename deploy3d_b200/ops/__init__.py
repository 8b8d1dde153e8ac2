"""Operator layer with the names and call signatures of ``deploy3d.symfun.ops``
(deploy3d/symfun/ops/__init__.py:1-5).

In the reference each operator is a ``torch.autograd.Function`` whose ``forward`` only allocates
zero tensors of the right shapes and whose ``symbolic`` emits a ``TRT_PluginV2`` node carrying the
plugin name and the packed ``data_s`` parameter blob.  Here each operator builds the *same* blob,
deserialises the plugin from it and enqueues it on the current CUDA stream, so the call returns the
real result.  ``data_s_*`` helpers expose the blob encoders (the wire format of the plugin boundary).
"""
from .spconv import (bev_densify, data_s_bev_densify, data_s_spconv_index, data_s_spconv_mm, spconv_index,
                     spconv_mm)
from .voxel_encoder import (cylinder_encoder, data_s_voxel_encoder, simple_mean_encoder)
from .point_voxel_mapping import (data_s_gather_back, data_s_scatter_to, gather_back, scatter_to)
from .decoder import data_s_yolox3d_decode, nms3d, yolox3d_decode

__all__ = ["spconv_index", "spconv_mm", "bev_densify", "simple_mean_encoder", "cylinder_encoder", "scatter_to",
           "gather_back", "nms3d", "yolox3d_decode", "data_s_yolox3d_decode", "data_s_spconv_index", "data_s_spconv_mm", "data_s_bev_densify",
           "data_s_voxel_encoder", "data_s_scatter_to", "data_s_gather_back"]
