"""Generates tests/golden/plugin_blobs.npz: the `data_s` blobs (and plugin name, version, number of outputs) that the
REFERENCE's own exporter writes, obtained by calling the `symbolic()` of every autograd Function under
deploy3d/symfun/ops with a recording stand-in for the ONNX graph, and the output shapes / dtypes its shape-only
`forward()` allocates for fixed input shapes.  Run where the reference checkout exists:

    python tests/golden/make_golden_blobs.py [/path/to/reference]

The reference's code predates numpy 1.24 (`np.bool`); the alias is restored for this script only.  The parameter
sets are listed in CASES so that the test can rebuild the same blobs with deploy3d_b200.ops.data_s_*."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

W = (np.arange(27 * 4 * 8, dtype=np.float32).reshape(27, 4, 8) / 100.0 - 3.0)
B = np.linspace(-1, 1, 8, dtype=np.float32)
CASES = [
    # (key, op class name, positional parameters after the tensor inputs)
    ("index_subm", "SPConvIdx3d", ((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), 20000, True, False)),
    ("index_down", "SPConvIdx3d", ((3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), 50000, False, False)),
    ("index_up", "SPConvIdx3d", ((3, 1, 3), (2, 1, 2), (1, 0, 1), (1, 2, 1), (0, 1, 0), 4321, False, True)),
    ("mm_bias", "SPConvMM", ((3, 3, 3), 4, 8, 1234, True, False, W, B)),
    ("mm_nobias_inverse", "SPConvMM", ((3, 3, 3), 4, 8, 99, False, True, W, None)),
    ("densify", "BEVDensify", (256,)),
    ("mean", "SimpleMeanEncoder", (60000,)),
    ("cylinder", "CylinderEncoder", (120000,)),
    ("scatter_max", "ScatterTo", (0,)),
    ("scatter_mean", "ScatterTo", (1,)),
    ("gather_fill", "GatherBack", (6.9,)),
    ("gather_keep", "GatherBack", (None,)),
    ("nms", "NMS3d", ()),
    ("decode", "YoloX3dDecode", (8, (0, 3, 7), 500)),
]
# tensor inputs of every op: (shape, dtype name); zero-element tensors carry spatial shapes, as in the reference
INPUTS = {
    "SPConvIdx3d": [((100, 4), "int32"), ((1,), "int32"), ((2, 0, 8, 16, 16), "int32")],
    "SPConvMM": [((100, 4), "float16"), ((1,), "int32"), ((1,), "int32"), ((3, 27 * 228), "int32"), ((1,), "int32")],
    "BEVDensify": [((100, 128), "float32"), ((100, 4), "int32"), ((1,), "int32"), ((2, 0, 2, 16, 16), "int32")],
    "SimpleMeanEncoder": [((500, 4), "float32"), ((500,), "int32"), ((6,), "float32"), ((2, 0, 8, 16, 16), "int32")],
    "CylinderEncoder": [((500, 4), "float32"), ((500,), "int32"), ((6,), "float32"), ((2, 0, 48, 36, 8), "int32")],
    "ScatterTo": [((500, 9), "float32"), ((500,), "int32"), ((64,), "int32")],
    "GatherBack": [((64, 9), "float32"), ((500,), "int32")],
    "NMS3d": [((2, 50), "float32"), ((2, 50, 7), "float32")],
    "YoloX3dDecode": [((2, 3, 32, 32), "float32"), ((2, 9, 32, 32), "float32"), ((6,), "float32")],
}
N_TENSOR_INPUTS = {k: len(v) for k, v in INPUTS.items()}


def make_inputs(cls):
    import torch
    return [torch.zeros(shape, dtype=getattr(torch, dt)) for shape, dt in INPUTS[cls]]


class RecordingGraph:
    """Stands in for torch._C.Graph: keeps the attributes of the one node a symbolic() emits."""

    def op(self, kind, *inputs, **attrs):
        self.kind, self.n_inputs, self.attrs = kind, len(inputs), attrs
        return None


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    # the reference checkout: argv[1], by default a directory `reference` beside this repository
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.abspath(os.path.join(here, "..", "..", "..", "reference"))
    np.bool = np.bool_  # removed from numpy; the reference's exporter still spells it this way
    sys.path.insert(0, ref)
    import deploy3d.symfun.ops as ops
    out = {}
    for key, cls, params in CASES:
        g = RecordingGraph()
        getattr(ops, cls).symbolic(g, *([None] * N_TENSOR_INPUTS[cls]), *params)
        assert g.kind == "TRT_PluginV2" and g.n_inputs == N_TENSOR_INPUTS[cls]
        out[key + "_data"] = np.frombuffer(g.attrs["data_s"], dtype=np.uint8).copy()
        out[key + "_name"] = np.frombuffer(g.attrs["name_s"], dtype=np.uint8).copy()
        out[key + "_version"] = np.frombuffer(g.attrs["version_s"], dtype=np.uint8).copy()
        out[key + "_outputs"] = np.int64(g.attrs["outputs"])
        # forward() of the reference's Function only allocates outputs of the right shape and dtype: record them
        res = getattr(ops, cls).forward(None, *make_inputs(cls), *params)
        res = res if isinstance(res, (tuple, list)) else (res,)
        assert len(res) == int(g.attrs["outputs"])
        for oi, t in enumerate(res):
            out["%s_out%d_shape" % (key, oi)] = np.array(list(t.shape), dtype=np.int64)
            out["%s_out%d_dtype" % (key, oi)] = np.frombuffer(str(t.dtype).encode(), dtype=np.uint8).copy()
    path = os.path.join(HERE, "plugin_blobs.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
