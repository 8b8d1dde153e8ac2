"""Whole-frame detection pipeline on one GPU: voxel encoder -> sparse backbone -> BEV densify, plus the
rotated-BEV NMS of the detection head -- the chain of plugins a deploy3d engine runs per frame
(deploy3d/symfun/models/lidar_detect.py:53-96 feeds points in and reads boxes out; the plugin chain
in between is what TensorRT enqueues).  Everything between the input copy and the output copy is
enqueued on one stream without host synchronisation and is captured into a CUDA graph.
"""
import numpy as np
import torch

from . import backbone, synth
from .ops import data_s_bev_densify, data_s_voxel_encoder
from .plugins import deserialize_plugin


def _roundup(v, m):
    return (int(v) + m - 1) // m * m


class DetectionPipeline:
    """CenterPoint-shaped (``kind='centerpoint'``) or SECOND-shaped (``kind='second'``) frame pipeline."""

    def __init__(self, kind="centerpoint", device="cuda:0", caps=None, kernel=0, n_class=10, topk=1000,
                 iou_threshold=0.2, dtype=torch.float16, n_pts=None, overlap_rulebooks=True, plugin_order=False,
                 regroup=False):
        self.kind, self.device, self.dtype = kind, torch.device(device), dtype
        # plugin order: one stream, nodes in ONNX order through the plugin-level entry points only (see SparseNet)
        self.plugin_order = plugin_order
        if kind == "centerpoint":
            frame = synth.config4_points()
            self.layers = backbone.voxel_res_backbone_8x(5)
        elif kind == "second":
            frame = synth.config3_points()
            self.layers = backbone.voxel_backbone_8x(4)
        else:
            raise ValueError(kind)
        self.n_pts, self.c_pts = frame["points"].shape
        if n_pts is not None:  # smaller point buffers (tests); the frame given to load_frame must have n_pts points
            self.n_pts = int(n_pts)
        self.spatial = frame["spatial_shape"]
        self.voxel_config = frame["voxel_config"]
        self.caps = caps or self.default_caps()
        dev = self.device
        with torch.cuda.device(dev):
            self.points = torch.zeros((self.n_pts, self.c_pts), dtype=torch.float32, device=dev)
            self.batch = torch.zeros(self.n_pts, dtype=torch.int32, device=dev)
            self.cfg = torch.from_numpy(self.voxel_config).to(dev)
            self.shape_tensor = torch.empty(self.spatial, dtype=torch.int32, device=dev)
            cap_in = self.caps["in"]
            self.vfe = deserialize_plugin("SimpleMeanEncoder", data_s_voxel_encoder(cap_in))
            self.vox_feats = torch.zeros((cap_in, self.c_pts), dtype=torch.float32, device=dev)
            self.vox_coors = torch.zeros((cap_in, 4), dtype=torch.int32, device=dev)
            self.vox_num = torch.zeros(1, dtype=torch.int32, device=dev)
            spatial_b = [self.spatial[0]] + list(self.spatial[2:])
            self.net = backbone.SparseNet(self.layers, spatial_b, self.caps, dtype=dtype, device=dev, kernel=kernel,
                                          overlap_rulebooks=overlap_rulebooks, plugin_order=plugin_order,
                                          regroup=regroup)
            # low-precision copy of the voxel features, zero-padded to the channel count the first layer runs with
            self.vox_feats_lp = torch.zeros((cap_in, self.net.in_channels), dtype=dtype, device=dev)
            self.net.set_input(self.vox_coors, self.vox_num)
            out = self.net.sets[self.net.out_set]
            self.out_shape = out["shape"]
            c_out = self.layers[-1].cout
            self.densify = deserialize_plugin("BEVDensify", data_s_bev_densify(c_out * self.out_shape[1]))
            self.out_shape_tensor = torch.empty([self.out_shape[0], 0] + self.out_shape[1:], dtype=torch.int32,
                                                device=dev)
            self.bev = torch.zeros((self.out_shape[0], c_out * self.out_shape[1], self.out_shape[2],
                                    self.out_shape[3]), dtype=dtype, device=dev)
            self.nms = deserialize_plugin("NMS3d", b"")
            self.nms.p.iou_threshold = iou_threshold
            self.scores = torch.zeros((n_class, topk), dtype=torch.float32, device=dev)
            self.boxes = torch.zeros((n_class, topk, 7), dtype=torch.float32, device=dev)
            self.nms_scores = torch.zeros((n_class, topk), dtype=torch.float32, device=dev)
        self.graph = None
        self.side = torch.cuda.Stream(device=self.device)

    def default_caps(self):
        """Static buffer sizes (the reference fixes them per model, e.g. [131072, 65536, 32768, 16384] in
        tests/cylinder/test_cylinder3d.py:391): generous here, tightened by calibrate()."""
        n = self.n_pts
        return {"in": n, "down2": 4 * n, "down3": 4 * n, "down4": 3 * n, "out": 3 * n}

    def calibrate(self, frames, margin=1.15):
        """Run `frames` once with generous buffers, read the voxel counts back and return tight caps."""
        peak = {}
        for f in frames:
            self.load_frame(f)
            self.enqueue()
            torch.cuda.synchronize(self.device)
            cnt = self.net.counts()
            cnt["in"] = int(self.vox_num.item())
            for k, v in cnt.items():
                if v >= self.caps[k]:
                    raise RuntimeError("voxel set %s filled its buffer (%d): raise the calibration caps" % (k, v))
                peak[k] = max(peak.get(k, 0), v)
        return {k: _roundup(v * margin + 256, 1024) for k, v in peak.items()}

    def load_frame(self, frame, boxes=None):
        """Synchronous convenience copy of one synthetic frame into the static input buffers."""
        self.points.copy_(torch.from_numpy(frame["points"]))
        self.batch.copy_(torch.from_numpy(frame["batch"]))
        if boxes is not None:
            self.scores.copy_(torch.from_numpy(boxes["scores"]))
            self.boxes.copy_(torch.from_numpy(boxes["boxes"]))

    def enqueue(self):
        """Enqueue one frame on the current stream (no host sync, no allocation after the first call).

        The NMS of the frame's candidate boxes is a parallel branch on a side stream: its inputs (decoded boxes) do
        not come from the backbone of the same frame in this workload, and it is a chain of two small, latency-bound
        kernels that fits beside the rulebook kernels.  (A deployed detector gets the same overlap by running the
        NMS of frame i beside the backbone of frame i+1.)  The branch joins before enqueue returns, so the caller
        still sees one stream; inside a CUDA graph capture it becomes a fork / join of the graph."""
        main = torch.cuda.current_stream(self.device)
        if not self.plugin_order:
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                self.nms.enqueue(self.scores, self.boxes, outputs=[self.nms_scores])
        if self.plugin_order or self.dtype == torch.float32:
            self.vfe.enqueue(self.points, self.batch, self.cfg, self.shape_tensor,
                             outputs=[self.vox_feats, self.vox_coors, self.vox_num])
            # fp32 -> fp16 reformat (TensorRT inserts this layer itself); padding columns stay zero
            self.vox_feats_lp[:, :self.c_pts].copy_(self.vox_feats)
        else:  # the encoder writes the half-precision, channel-padded copy itself
            self.vfe.enqueue_lp(self.points, self.batch, self.cfg, self.shape_tensor,
                                outputs=[self.vox_feats, self.vox_coors, self.vox_num], lp_feats=self.vox_feats_lp)
        feats, coors, num = self.net.forward(self.vox_feats_lp)
        self.densify.enqueue(feats, coors, num, self.out_shape_tensor, outputs=[self.bev])
        if self.plugin_order:
            self.nms.enqueue(self.scores, self.boxes, outputs=[self.nms_scores])
        else:
            main.wait_stream(self.side)
        return feats, coors, num

    def capture(self):
        """Capture enqueue() into a CUDA graph (after a warm-up call so every workspace exists)."""
        with torch.cuda.device(self.device):
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self.enqueue()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._graph_out = self.enqueue()
        return self.graph

    def replay(self):
        self.graph.replay()

    def buffer_bytes(self):
        """Bytes of every static buffer a frame touches (inputs, rulebooks, tables, activations, workspaces)."""
        total = 0
        seen = set()

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen and t.numel():
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        for t in (self.points, self.batch, self.vox_feats, self.vox_coors, self.vox_feats_lp, self.bev, self.boxes,
                  self.scores, self.nms_scores, self.vfe._workspace, self.densify._workspace, self.nms._workspace):
            add(t)
        for rb in self.net.rulebooks.values():
            for t in (rb.index, rb.table_fwd, rb.table_inv, rb.plugin._workspace):
                add(t)
        for _, buf, _ in self.net.mm:
            add(buf)
        for s in self.net.sets.values():
            add(s["coors"])
        return total


class SegmentationPipeline:
    """Cylinder3D-shaped frame pipeline: CylinderEncoder -> ScatterTo (max) -> asymmetric encoder-decoder sparse
    network with inverse convolutions -> GatherBack to per-point logits (the op chain of
    tests/cylinder/test_cylinder3d.py:275-325).  ``net='cylinder3d'`` is the network of benchmark config 5 (3x1x3 /
    1x3x3 SubM blocks, channels 32 / 64 / 128 / 256, 20 classes); ``net='unet'`` a small 3x3x3 encoder-decoder."""

    def __init__(self, device="cuda:0", n_pts=120000, caps=None, n_class=None, dtype=torch.float16, kernel=0,
                 net="cylinder3d", overlap_rulebooks=True, regroup=False):
        from .ops import data_s_gather_back, data_s_scatter_to
        frame = synth.config5_points()
        self.device, self.dtype, self.n_pts = torch.device(device), dtype, int(n_pts)
        self.c_pts = frame["points"].shape[1]
        self.spatial = frame["spatial_shape"]
        self.cylinder_config = frame["cylinder_config"]
        if net == "cylinder3d":
            self.n_class = n_class or 20
            self.layers = backbone.cylinder3d(self.c_pts + 5, self.n_class)
        else:
            self.n_class = n_class or 16
            self.layers = backbone.seg_unet(self.c_pts + 5, self.n_class)
        n_class = self.n_class
        self.set_names = ["in"] + [L.key for L in self.layers if L.kind == "conv"]
        self.caps = caps or {k: self.n_pts for k in self.set_names}
        dev = self.device
        with torch.cuda.device(dev):
            cap = self.caps["in"]
            self.points = torch.zeros((self.n_pts, self.c_pts), dtype=torch.float32, device=dev)
            self.batch = torch.zeros(self.n_pts, dtype=torch.int32, device=dev)
            self.cfg = torch.from_numpy(self.cylinder_config).to(dev)
            self.shape_tensor = torch.empty(self.spatial, dtype=torch.int32, device=dev)
            self.encoder = deserialize_plugin("CylinderEncoder", data_s_voxel_encoder(cap))
            self.pts_feats = torch.zeros((self.n_pts, self.c_pts + 5), dtype=torch.float32, device=dev)
            self.scatter_index = torch.zeros(self.n_pts, dtype=torch.int32, device=dev)
            self.scatter_count = torch.zeros(cap, dtype=torch.int32, device=dev)
            self.vox_coors = torch.zeros((cap, 4), dtype=torch.int32, device=dev)
            self.vox_num = torch.zeros(1, dtype=torch.int32, device=dev)
            self.scatter = deserialize_plugin("ScatterTo", data_s_scatter_to(0))
            self.vox_feats = torch.zeros((cap, self.c_pts + 5), dtype=torch.float32, device=dev)
            spatial_b = [self.spatial[0]] + list(self.spatial[2:])
            self.net = backbone.SparseNet(self.layers, spatial_b, self.caps, dtype=dtype, device=dev, kernel=kernel,
                                          overlap_rulebooks=overlap_rulebooks, regroup=regroup)
            self.vox_feats_lp = torch.zeros((cap, self.net.in_channels), dtype=dtype, device=dev)
            self.net.set_input(self.vox_coors, self.vox_num)
            self.gather = deserialize_plugin("GatherBack", data_s_gather_back(0.0))
            # GatherBack reads the half-precision network output and writes float logits
            self.logits = torch.zeros((self.n_pts, n_class), dtype=torch.float32, device=dev)
            self.labels = torch.zeros(self.n_pts, dtype=torch.int32, device=dev)
        self.graph = None

    def load_frame(self, frame):
        self.points.copy_(torch.from_numpy(frame["points"]))
        self.batch.copy_(torch.from_numpy(frame["batch"]))

    def calibrate(self, frames, margin=1.15):
        """Run `frames` once with generous buffers, read the voxel counts back and return tight caps."""
        peak = {}
        for f in frames:
            self.load_frame(f)
            self.enqueue()
            torch.cuda.synchronize(self.device)
            cnt = self.net.counts()
            cnt["in"] = int(self.vox_num.item())
            for k, v in cnt.items():
                if v >= self.caps[k]:
                    raise RuntimeError("voxel set %s filled its buffer (%d): raise the calibration caps" % (k, v))
                peak[k] = max(peak.get(k, 0), v)
        return {k: _roundup(v * margin + 256, 1024) for k, v in peak.items()}

    def enqueue(self):
        """One frame on the current stream: no host synchronisation, no allocation by this library (the
        element-wise graph ops between plugins are torch's)."""
        self.encoder.enqueue(self.points, self.batch, self.cfg, self.shape_tensor,
                             outputs=[self.pts_feats, self.scatter_index, self.scatter_count, self.vox_coors,
                                      self.vox_num])
        self.scatter.enqueue(self.pts_feats, self.scatter_index, self.scatter_count, outputs=[self.vox_feats])
        self.vox_feats_lp[:, :self.c_pts + 5].copy_(self.vox_feats)
        feats, _, _ = self.net.forward(self.vox_feats_lp)
        self.gather.enqueue(feats, self.scatter_index, outputs=[self.logits])
        self.labels.copy_(torch.argmax(self.logits, dim=1))  # the label pass of the reference (test_cylinder3d.py:322)
        return self.logits

    def capture(self):
        """Capture enqueue() into a CUDA graph (after a warm-up call so every workspace exists)."""
        with torch.cuda.device(self.device):
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self.enqueue()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.enqueue()
        return self.graph

    def replay(self):
        self.graph.replay()
