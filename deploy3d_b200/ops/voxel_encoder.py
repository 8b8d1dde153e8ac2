"""``simple_mean_encoder``, ``cylinder_encoder`` (deploy3d/symfun/ops/voxel_encoder/*.py)."""
import numpy as np

from .spconv import _plugin


def data_s_voxel_encoder(max_num_act_out):
    return np.array([max_num_act_out], dtype=np.int32).tobytes()


def simple_mean_encoder(batch_point_feats, batch_indices, voxel_config, in_spatial_shape, max_num_act_out):
    """Returns (out_feats, out_coors, num_act_out) (deploy3d/symfun/ops/voxel_encoder/simple_mean.py:21-33)."""
    plug = _plugin("SimpleMeanEncoder", data_s_voxel_encoder(max_num_act_out))
    return plug.enqueue(batch_point_feats, batch_indices, voxel_config, in_spatial_shape)


def cylinder_encoder(batch_point_feats, batch_indices, cylinder_config, in_spatial_shape, max_num_act_out):
    """Returns (pts_feats, scatter_to, scatter_count, out_coors, num_act_out)
    (deploy3d/symfun/ops/voxel_encoder/cylinder.py:23-37)."""
    plug = _plugin("CylinderEncoder", data_s_voxel_encoder(max_num_act_out))
    return plug.enqueue(batch_point_feats, batch_indices, cylinder_config, in_spatial_shape)
