"""Sparse backbones composed from the plugins, the way the reference's tests compose them
(tests/cylinder/test_cylinder3d.py:11-99: one SPConvIdx per ``indice_key`` shared by several SPConvMM
layers, batch-norm folded into weight and bias, activation after the plugin).

A ``SparseNet`` is built once ("engine build": plugin handles, weights uploaded, every buffer and
workspace allocated at its static maximum size, exactly as TensorRT would own them) and then run
frame after frame with no allocation and no host synchronisation, so a whole frame can be captured
in a CUDA graph.  Layers that share a rulebook also share one output-stationary neighbour table.
"""
import numpy as np
import torch

from . import synth
from .ops import data_s_spconv_index, data_s_spconv_mm
from .plugins import SPConvMMPlugin, deserialize_plugin


class Layer:
    """One sparse convolution.

    kind      'subm' | 'conv' (strided, creates a new voxel set) | 'inverse' (back to the inputs of `key`'s conv) |
              'ew' (an element-wise graph op between plugins: `ew` = (name, [saved tags]); TensorRT-native layers in
              the reference's graph, plain tensor ops here)
    key       rulebook name (``indice_key``); the first layer naming a key builds it
    residual  name of a saved activation added to the result (fused epilogue), or None
    act_first the ReLU comes before the residual add (sum of two activated branches) instead of after it
    save      name under which the output is kept for a later residual / skip connection
    source    name of the saved activation the layer reads (default: the previous layer's output)
    """

    def __init__(self, kind, key, cin, cout, ksize=(3, 3, 3), stride=(1, 1, 1), padding=None, relu=True,
                 residual=None, save=None, source=None, act_first=False, ew=None):
        self.kind, self.key, self.cin, self.cout = kind, key, cin, cout
        self.ksize, self.stride = tuple(ksize), tuple(stride)
        self.padding = tuple(k // 2 for k in ksize) if padding is None else tuple(padding)
        self.relu, self.residual, self.save, self.source = relu, residual, save, source
        self.act_first, self.ew = act_first, ew

    @property
    def relu_mode(self):
        """The `relu` field of d3d_spconv_mm_epilogue."""
        return 0 if not self.relu else (2 if self.act_first else 1)


def ew_apply(name, xs, xp):
    """The element-wise graph ops of the Cylinder3D-shaped network, for torch tensors (xp = torch) and numpy arrays
    (xp = numpy) alike, in fp32: 'recon' = (sigmoid(a) + sigmoid(b) + sigmoid(c)) * x, the ReconBlock of
    tests/cylinder/test_cylinder3d.py:181-205; 'concat' = channel concatenation (:262-263)."""
    if name == "recon":
        a, b, c, x = xs
        sig = (lambda t: 1.0 / (1.0 + xp.exp(-t)))
        return (sig(a) + sig(b) + sig(c)) * x
    if name == "concat":
        return xp.cat(xs, 1) if hasattr(xp, "cat") else xp.concatenate(xs, 1)
    raise ValueError(name)


def res_block(key, c, tag):
    """SparseBasicBlock: relu(conv2(relu(conv1(x))) + x), both SubM over the same rulebook."""
    return [Layer("subm", key, c, c, save=None, source=None, relu=True, residual=None),
            Layer("subm", key, c, c, relu=True, residual=tag)]


def voxel_res_backbone_8x(cin):
    """CenterPoint-shaped VoxelResBackBone8x, channels 16/32/64/128: input SubM, then per stage a strided conv
    (stage 1 has none) followed by two residual blocks, then the (3,1,1)/(2,1,1) output conv."""
    L = [Layer("subm", "subm1", cin, 16, save="s1")]
    for i in range(2):
        blk = res_block("subm1", 16, "s1")
        blk[1].save = "s1"
        L += blk
    chans = [16, 32, 64, 128]
    pads = [None, (1, 1, 1), (1, 1, 1), (0, 1, 1)]
    for s in range(1, 4):
        tag = "s%d" % (s + 1)
        L.append(Layer("conv", "down%d" % (s + 1), chans[s - 1], chans[s], stride=(2, 2, 2), padding=pads[s], save=tag))
        for i in range(2):
            blk = res_block("subm%d" % (s + 1), chans[s], tag)
            blk[1].save = tag
            L += blk
    L.append(Layer("conv", "out", 128, 128, ksize=(3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0)))
    return L


def voxel_backbone_8x(cin):
    """SECOND-shaped VoxelBackBone8x, channels 16/32/64/64, ending in the (3,1,1)/(2,1,1) conv to 128."""
    L = [Layer("subm", "subm1", cin, 16), Layer("subm", "subm1", 16, 16)]
    chans = [16, 32, 64, 64]
    pads = [None, (1, 1, 1), (1, 1, 1), (0, 1, 1)]
    for s in range(1, 4):
        L.append(Layer("conv", "down%d" % (s + 1), chans[s - 1], chans[s], stride=(2, 2, 2), padding=pads[s]))
        L.append(Layer("subm", "subm%d" % (s + 1), chans[s], chans[s]))
        L.append(Layer("subm", "subm%d" % (s + 1), chans[s], chans[s]))
    L.append(Layer("conv", "out", 64, 128, ksize=(3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0)))
    return L


def seg_unet(cin, n_class=16):
    """Cylinder3D-shaped encoder-decoder for per-point segmentation (the composition of the reference's
    tests/cylinder/test_cylinder3d.py:11-99: SubM blocks, strided downsampling, and upsampling by the INVERSE of
    the same rulebook with a skip connection added before the ReLU).  Output is on the input voxel set."""
    return [
        Layer("subm", "s0", cin, 32, save="e0"),
        Layer("conv", "d1", 32, 64, stride=(2, 2, 2), padding=(1, 1, 1)),
        Layer("subm", "s1", 64, 64, save="e1"),
        Layer("conv", "d2", 64, 128, stride=(2, 2, 2), padding=(1, 1, 1)),
        Layer("subm", "s2", 128, 128),
        Layer("inverse", "d2", 128, 64, residual="e1"),
        Layer("subm", "s1", 64, 64),
        Layer("inverse", "d1", 64, 32, residual="e0"),
        Layer("subm", "s0", 32, n_class, relu=False),
    ]


def cylinder3d(cin, n_class=20, init=32):
    """Cylinder3D-shaped asymmetric encoder-decoder, channels init / 2 init / 4 init / 8 init (32 / 64 / 128 / 256),
    composed as the reference composes it (tests/cylinder/test_cylinder3d.py:100-272): ResContextBlock, three
    ResBlocks (two branches of 3x1x3 / 1x3x3 SubM convolutions over shared rulebooks, summed, then a strided
    pooling convolution), three UpBlocks (3x3x3 SubM, inverse of the matching pooling convolution, skip connection,
    1x3x3 / 3x1x3 / 3x3x3 SubM), ReconBlock (3x1x1, 1x3x1, 1x1x3 with sigmoid, summed, times the input), channel
    concatenation and the 3x3x3 logits convolution.  Batch norm is folded into weight and bias (:24-37); the
    activation is ReLU (the plugin has none: it is a graph op after it, :91-92)."""
    k133, k313 = (1, 3, 3), (3, 1, 3)
    c = init
    L = [  # ResContextBlock: shortcut = conv1_2(conv1(x)); out = conv3(conv2(x)) + shortcut
        Layer("subm", "res2_1", cin, c, ksize=k133, source="input"),
        Layer("subm", "res1_1", c, c, ksize=k313, save="ctx_short"),
        Layer("subm", "res1_1", cin, c, ksize=k313, source="input"),
        Layer("subm", "res2_1", c, c, ksize=k133, residual="ctx_short", act_first=True, save="down0"),
    ]
    strides = [(2, 2, 2), (2, 2, 2), (2, 2, 1)]
    for i in range(3):  # ResBlock i at stride 2^i: resA = conv3(conv2(x)) + conv1_2(conv1(x)); resB = pool(resA)
        s = 1 << i
        cout, src = 2 * c, "down%d" % i
        L += [
            Layer("subm", "res1_%d" % s, c, cout, ksize=k313, source=src),
            Layer("subm", "res2_%d" % s, cout, cout, ksize=k133, save="short%d" % i),
            Layer("subm", "res2_%d" % s, c, cout, ksize=k133, source=src),
            Layer("subm", "res1_%d" % s, cout, cout, ksize=k313, residual="short%d" % i, act_first=True,
                  save="skip%d" % i),
            Layer("conv", "res_pool_%d" % s, cout, cout, stride=strides[i], padding=(1, 1, 1), relu=False,
                  save="down%d" % (i + 1)),
        ]
        c = cout
    for i in range(3):  # UpBlock at stride 4, 2, 1: up = inverse_pool(trans(x)) + skip; conv1, conv2, conv3
        lvl = 2 - i
        s = 1 << lvl
        cout = c if i == 0 else c // 2
        L += [
            Layer("subm", "trans_dilao_%d" % s, c, cout),
            Layer("inverse", "res_pool_%d" % s, cout, cout, relu=False, residual="skip%d" % lvl),
            Layer("subm", "res2_%d" % s, cout, cout, ksize=k133),
            Layer("subm", "res1_%d" % s, cout, cout, ksize=k313),
            Layer("subm", "up3_%d" % s, cout, cout, save="up%d" % i),
        ]
        c = cout
    L += [  # ReconBlock, concatenation, logits
        Layer("subm", "rec1", c, c, ksize=(3, 1, 1), relu=False, source="up2", save="rec_a"),
        Layer("subm", "rec1_2", c, c, ksize=(1, 3, 1), relu=False, source="up2", save="rec_b"),
        Layer("subm", "rec1_3", c, c, ksize=(1, 1, 3), relu=False, source="up2", save="rec_c"),
        Layer("ew", None, c, c, ew=("recon", ["rec_a", "rec_b", "rec_c", "up2"]), save="recon"),
        Layer("ew", None, c, 2 * c, ew=("concat", ["recon", "up2"])),
        Layer("subm", "logits", 2 * c, n_class, relu=False),
    ]
    return L


def make_weights(layers, seed=0):
    """Seeded Kaiming weights [kVol, Cin, Cout] and small biases (batch-norm folded) for every layer, in order
    (None for the element-wise graph ops)."""
    rng = np.random.Generator(np.random.PCG64(4242 + seed))
    out = []
    for L in layers:
        if L.kind == "ew":
            out.append(None)
            continue
        kvol = int(np.prod(L.ksize))
        w = synth.kaiming_weight(rng, kvol, L.cin, L.cout)
        b = (rng.standard_normal(L.cout) * 0.05).astype(np.float32)
        out.append((w, b))
    return out


class _Rulebook:
    pass


class SparseNet:
    """Executable sparse network with static buffers.

    layers      list of Layer
    spatial     [B, Z, Y, X] of the input voxel grid
    caps        dict voxel-set name -> maximum active voxels ('in' for the input set, otherwise the key of the
                'conv' layer that creates the set)
    The network input is available to later layers under the tag 'input'.  A first layer with 4, 5 or 9 input
    channels runs with its input zero-padded to 16 channels (zero weight rows) and a last layer whose output
    channel count is not a multiple of 16 with zero-padded output channels, which makes both eligible for the
    tensor-core kernel; `forward` returns the un-padded view.
    """

    def __init__(self, layers, spatial, caps, dtype=torch.float16, device="cuda:0", seed=0, kernel=0,
                 pad_input=True, overlap_rulebooks=False, plugin_order=False, regroup=False):
        self.layers, self.device, self.dtype = layers, torch.device(device), dtype
        # regroup: every neighbour table is rebuilt with its outputs grouped by offset mask (same results, fewer
        # (tile, offset) blocks for the convolutions to walk); never in plugin order, where a table serves one layer
        self.regroup = regroup and not plugin_order
        # plugin order: what a TensorRT engine built from the reference's ONNX graph executes -- one stream, every
        # SPConvMM node through the plugin-level enqueue (which rebuilds its neighbour table in its own workspace,
        # trt/spconv/mm_trt.cu:149-205 has no state shared between nodes), ReLU / residual add as separate
        # element-wise layers after the plugin (tests/cylinder/test_cylinder3d.py:91-92)
        self.plugin_order = plugin_order
        overlap_rulebooks = overlap_rulebooks and not plugin_order
        self.overlap_rulebooks = overlap_rulebooks
        self.side = torch.cuda.Stream(device=self.device) if overlap_rulebooks else None
        self.side_subm = torch.cuda.Stream(device=self.device) if overlap_rulebooks else None
        self.kernel = kernel
        weights = make_weights(layers, seed)
        self.rulebooks = {}
        self.mm = []
        self.sets = {"in": dict(cap=int(caps["in"]), shape=[int(v) for v in spatial], coors=None, num=None)}
        cur = "in"
        set_of_tag = {"input": "in"}
        lp = dtype != torch.float32
        first_cin = next(L.cin for L in layers if L.kind != "ew")
        self.in_channels = (first_cin + 15) // 16 * 16 if (lp and pad_input and first_cin % 16) else first_cin
        self.out_channels = layers[-1].cout
        with torch.cuda.device(self.device):
            for li, L in enumerate(layers):
                if L.kind == "ew":
                    cur = set_of_tag[L.ew[1][0]]
                    out_buf = torch.zeros((self.sets[cur]["cap"], L.cout), dtype=dtype, device=self.device)
                    self.mm.append((None, out_buf, cur))
                    if L.save:
                        set_of_tag[L.save] = cur
                    continue
                if L.source is not None:
                    cur = set_of_tag[L.source]
                src = self.sets[cur]
                if L.key not in self.rulebooks:
                    assert L.kind != "inverse", "an inverse layer needs the rulebook of its conv"
                    rb = _Rulebook()
                    rb.kind, rb.in_set, rb.ksize = L.kind, cur, L.ksize
                    # SubM with an odd kernel and 'same' padding: offsets k and kVol-1-k mirror each other
                    rb.mirror = (L.kind == "subm" and all(k % 2 == 1 for k in L.ksize) and
                                 tuple(L.padding) == tuple(k // 2 for k in L.ksize))
                    rb.kvol = int(np.prod(L.ksize))
                    subm = L.kind == "subm"
                    if subm:
                        rb.out_set = cur
                    else:
                        shp = src["shape"]
                        oshape = [shp[0]] + [(shp[d + 1] + 2 * L.padding[d] - (L.ksize[d] - 1) - 1) // L.stride[d] + 1
                                             for d in range(3)]
                        cap = int(caps[L.key])
                        self.sets[L.key] = dict(cap=cap, shape=oshape, coors=None, num=None)
                        rb.out_set = L.key
                    out = self.sets[rb.out_set]
                    rb.plugin = deserialize_plugin("SPConvIdx3d", data_s_spconv_index(
                        L.ksize, L.stride, L.padding, (1, 1, 1), (0, 0, 0), out["cap"], subm, False))
                    rb.shape_tensor = torch.empty([src["shape"][0], 0] + src["shape"][1:], dtype=torch.int32,
                                                  device=self.device)
                    row_len = rb.kvol * (src["cap"] + 128)
                    rb.out_shape_tensor = torch.empty([out["shape"][0], 0] + out["shape"][1:], dtype=torch.int32,
                                                      device=self.device)
                    rb.index = torch.empty((3, row_len), dtype=torch.int32, device=self.device)
                    rb.num_index = torch.zeros(1, dtype=torch.int32, device=self.device)
                    if not subm:
                        out["coors"] = torch.zeros((out["cap"], 4), dtype=torch.int32, device=self.device)
                        out["num"] = torch.zeros(1, dtype=torch.int32, device=self.device)
                    rb.table_fwd = None if plugin_order else torch.empty(
                        max(SPConvMMPlugin.table_bytes(rb.kvol, out["cap"]), 16), dtype=torch.uint8,
                        device=self.device)
                    rb.table_inv = None
                    rb.raw_fwd = rb.raw_inv = rb.scratch_fwd = rb.scratch_inv = None
                    rb.regroup = self.regroup and rb.kvol <= 32
                    if rb.regroup:  # the builders write the plain table, the layers read the regrouped one
                        rb.raw_fwd = torch.empty_like(rb.table_fwd)
                        rb.scratch_fwd = torch.empty(
                            max(SPConvMMPlugin.regroup_scratch_bytes(rb.kvol, out["cap"]), 16), dtype=torch.uint8,
                            device=self.device)
                    # the net owns index, workspace and tables for its whole life: stale-padding-only refills, and
                    # the table of a mirror-symmetric SubM rulebook straight from the probe kernel
                    rb.calls = 0
                    rb.fused_table = subm and not plugin_order and rb.plugin.subm_table_ok()
                    self.rulebooks[L.key] = rb
                rb = self.rulebooks[L.key]
                if L.kind == "inverse":
                    out_set, in_set = rb.in_set, rb.out_set
                    if rb.table_inv is None and not plugin_order:
                        rb.table_inv = torch.empty(
                            max(SPConvMMPlugin.table_bytes(rb.kvol, self.sets[out_set]["cap"]), 16),
                            dtype=torch.uint8, device=self.device)
                        if rb.regroup:
                            rb.raw_inv = torch.empty_like(rb.table_inv)
                            rb.scratch_inv = torch.empty(
                                max(SPConvMMPlugin.regroup_scratch_bytes(rb.kvol, self.sets[out_set]["cap"]), 16),
                                dtype=torch.uint8, device=self.device)
                else:
                    out_set, in_set = rb.out_set, rb.in_set
                assert in_set == cur, "layer %d expects voxel set %s but the data is on %s" % (li, in_set, cur)
                w, b = weights[li]
                cin, cout = L.cin, L.cout
                reads_input = (li == 0 and L.source is None) or L.source == "input"
                if reads_input and cin != self.in_channels:
                    wp = np.zeros((w.shape[0], self.in_channels, w.shape[2]), dtype=np.float32)
                    wp[:, :cin] = w
                    w, cin = wp, self.in_channels
                if li == len(layers) - 1 and lp and cout % 16:
                    cout = (cout + 15) // 16 * 16
                    wp = np.zeros((w.shape[0], w.shape[1], cout), dtype=np.float32)
                    wp[:, :, :L.cout] = w
                    bp = np.zeros(cout, dtype=np.float32)
                    bp[:L.cout] = b
                    w, b = wp, bp
                plug = deserialize_plugin("SPConvMM", data_s_spconv_mm(
                    L.ksize, cin, cout, self.sets[out_set]["cap"], L.kind == "subm", L.kind == "inverse", w, b))
                plug.configure(dtype)
                plug.set_kernel(kernel)
                # single-stream execution: the next layer's prologue overlaps this layer's tail; with the rulebook
                # chain on a side stream its kernels fill those tails instead (measured: 1 % better per frame)
                plug.set_dependent_launch(not overlap_rulebooks)
                out_buf = torch.zeros((self.sets[out_set]["cap"], cout), dtype=dtype, device=self.device)
                self.mm.append((plug, out_buf, out_set))
                cur = out_set
                if L.save:
                    set_of_tag[L.save] = cur
            self.out_set = cur

    def set_input(self, coors, num):
        self.sets["in"]["coors"], self.sets["in"]["num"] = coors, num

    def _build_rulebook(self, rb):
        src, dst = self.sets[rb.in_set], self.sets[rb.out_set]
        if self.plugin_order:  # the plain plugin entry point; every SPConvMM node builds its own table
            outs = [rb.index, rb.num_index] if rb.kind == "subm" else \
                [rb.index, rb.num_index, dst["coors"], dst["num"], rb.out_shape_tensor]
            rb.plugin.enqueue(src["coors"], src["num"], rb.shape_tensor, outputs=outs)
            return
        first = rb.calls == 0
        rb.calls += 1
        plain_fwd = rb.raw_fwd if rb.regroup else rb.table_fwd
        if rb.kind == "subm":
            rb.plugin.enqueue_ex(src["coors"], src["num"], rb.shape_tensor, outputs=[rb.index, rb.num_index],
                                 persistent=True, first_call=first,
                                 subm_table=plain_fwd if rb.fused_table else None)
        else:
            rb.plugin.enqueue_ex(src["coors"], src["num"], rb.shape_tensor,
                                 outputs=[rb.index, rb.num_index, dst["coors"], dst["num"], rb.out_shape_tensor],
                                 persistent=True, first_call=first)
        if not rb.fused_table:
            SPConvMMPlugin.prepare(rb.kvol, False, dst["cap"], rb.index, rb.num_index, table=plain_fwd,
                                   mirror=rb.mirror)
        if rb.regroup:
            SPConvMMPlugin.regroup(rb.kvol, dst["cap"], plain_fwd, rb.table_fwd, rb.scratch_fwd)
        if rb.table_inv is not None:
            SPConvMMPlugin.prepare(rb.kvol, True, src["cap"], rb.index, rb.num_index,
                                   table=rb.raw_inv if rb.regroup else rb.table_inv)
            if rb.regroup:
                SPConvMMPlugin.regroup(rb.kvol, src["cap"], rb.raw_inv, rb.table_inv, rb.scratch_inv)

    def forward(self, feats):
        """feats [cap_in, Cin] in the net dtype; coordinates / count as given to set_input.  Returns
        (out_feats, out_coors, num_act_out); every tensor is a static buffer of the net.

        Rulebooks and neighbour tables depend on coordinates only, never on features, so with `overlap_rulebooks`
        the chains of them are enqueued on two side streams ahead of the convolutions; a layer waits for the event
        of its own rulebook.  Inside a CUDA graph capture these become further branches of the graph."""
        main = torch.cuda.current_stream(self.device)
        ready = {}
        if self.overlap_rulebooks:
            # two chains: the strided rulebooks follow each other (each creates the voxel set of the next); the SubM
            # rulebook of a level needs only that level's coordinates, so it runs beside the next strided one.
            # (A third stream for the strided rulebooks' neighbour tables measured no further gain.)
            self.side.wait_stream(main)
            self.side_subm.wait_stream(main)
            done = set()
            for L in self.layers:
                if L.kind == "ew" or L.key in done:
                    continue
                done.add(L.key)
                rb = self.rulebooks[L.key]
                stream = self.side_subm if rb.kind == "subm" else self.side
                with torch.cuda.stream(stream):
                    # rb.in_set is named after the strided rulebook that wrote its coordinates ('in': the caller)
                    if rb.kind == "subm" and rb.in_set in ready:
                        stream.wait_event(ready[rb.in_set])
                    self._build_rulebook(rb)
                    ev = torch.cuda.Event()
                    ev.record(stream)
                    ready[L.key] = ev
        built = set()
        saved = {"input": feats}
        x = feats
        for L, (plug, out_buf, out_set) in zip(self.layers, self.mm):
            if L.kind == "ew":  # element-wise graph op between plugins, in fp32 like the CPU restatement
                y = ew_apply(L.ew[0], [saved[t].float() for t in L.ew[1]], torch)
                out_buf.copy_(y)
                x = out_buf
                if L.save:
                    saved[L.save] = x
                continue
            if L.source is not None:
                x = saved[L.source]
            rb = self.rulebooks[L.key]
            if L.key not in built:
                if self.overlap_rulebooks:
                    main.wait_event(ready[L.key])
                else:
                    self._build_rulebook(rb)
                built.add(L.key)
            res = saved[L.residual] if L.residual else None
            if self.plugin_order:
                in_set = rb.out_set if L.kind == "inverse" else rb.in_set
                plug.enqueue(x, self.sets[in_set]["num"], self.sets[out_set]["num"], rb.index, rb.num_index,
                             outputs=[out_buf])
                if L.relu and L.act_first:
                    out_buf.relu_()
                if res is not None:
                    out_buf.add_(res)
                if L.relu and not L.act_first:
                    out_buf.relu_()
                x = out_buf
            else:
                table = rb.table_inv if L.kind == "inverse" else rb.table_fwd
                x = plug.run(x, self.sets[out_set]["num"], table, out=out_buf, relu=L.relu_mode, residual=res,
                             regrouped=rb.regroup)
            if L.save:
                saved[L.save] = x
        if self.overlap_rulebooks:
            main.wait_stream(self.side)
            main.wait_stream(self.side_subm)
        o = self.sets[self.out_set]
        if x.shape[1] != self.out_channels:
            x = x[:, :self.out_channels]
        return x, o["coors"], o["num"]

    def counts(self):
        """Active voxels of every set (host sync; for calibration and reporting only)."""
        return {k: int(v["num"].item()) for k, v in self.sets.items() if v["num"] is not None}

    def layer_work(self):
        """Per convolution layer: (Cin, Cout, kVol, M, pairs P) after a forward pass (host sync)."""
        out = []
        pairs = {}
        for L, (plug, _, out_set) in zip(self.layers, self.mm):
            if L.kind == "ew":
                continue
            rb = self.rulebooks[L.key]
            if L.key not in pairs:
                k = rb.index[2, :int(rb.num_index.item())]
                pairs[L.key] = int((k >= 0).sum().item())
            out.append((plug.p.in_channels, plug.p.out_channels, rb.kvol, int(self.sets[out_set]["num"].item()),
                        pairs[L.key]))
        return out
