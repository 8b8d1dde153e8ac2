"""``scatter_to``, ``gather_back`` (deploy3d/symfun/ops/point_voxel_mapping/*.py)."""
import numpy as np

from .spconv import _plugin


def data_s_scatter_to(reduce_type):
    return np.array([reduce_type], dtype=np.int8).tobytes()


def scatter_to(batch_point_feats, scatter_to, scatter_count, reduce_type):
    """reduce_type 0: max, otherwise mean (deploy3d/symfun/ops/point_voxel_mapping/scatter_to.py:19-28)."""
    plug = _plugin("ScatterTo", data_s_scatter_to(reduce_type))
    return plug.enqueue(batch_point_feats, scatter_to, scatter_count)[0]


def data_s_gather_back(fill_val=None):
    data = np.array([fill_val is not None], dtype=np.bool_).tobytes()
    # without a fill value the exporter serialises None as float32, i.e. NaN; the flag byte is what counts
    data += np.array([np.nan if fill_val is None else fill_val], dtype=np.float32).tobytes()
    return data


def gather_back(reduces_feats, scatter_to, fill_val=None, out=None):
    """Rows whose index is negative are filled with ``fill_val`` when given, otherwise left untouched
    (deploy3d/symfun/ops/point_voxel_mapping/gather_back.py:19-27)."""
    plug = _plugin("GatherBack", data_s_gather_back(fill_val))
    return plug.enqueue(reduces_feats, scatter_to, outputs=None if out is None else [out])[0]
