"""Builds (g++, no TensorRT needed) and loads the test harness around the TensorRT plugin shells:
tests/trt_stub/harness.cpp compiles deploy3d_b200/csrc/trt/deploy3d_trt_plugins.cpp against the stand-in header
tests/trt_stub/NvInfer.h and links it to libdeploy3d_b200.so."""
import ctypes
import os
import shutil
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STUB = os.path.join(ROOT, "tests", "trt_stub")
OUT = os.path.join(STUB, "_build", "libd3d_trt_shells_test.so")
SOURCES = [os.path.join(STUB, "harness.cpp"), os.path.join(STUB, "NvInfer.h"),
           os.path.join(ROOT, "deploy3d_b200", "csrc", "trt", "deploy3d_trt_plugins.cpp"),
           os.path.join(ROOT, "include", "deploy3d_b200.h")]


class Desc(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("nb_dims", ctypes.c_int32), ("dims", ctypes.c_int64 * 8)]


def build(force=False):
    from deploy3d_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from deploy3d_b200 import build as lib_build
        lib_build.build()
    stale = force or not os.path.exists(OUT) or any(os.path.getmtime(s) > os.path.getmtime(OUT) for s in SOURCES)
    if stale:
        gxx = shutil.which("g++")
        if gxx is None:
            raise RuntimeError("g++ not found: cannot compile the TensorRT plugin shells")
        os.makedirs(os.path.dirname(OUT), exist_ok=True)
        libdir = os.path.dirname(_lib.LIB_PATH)
        cmd = [gxx, "-std=c++14", "-O1", "-Wall", "-Werror", "-fPIC", "-shared", SOURCES[0], "-I" + STUB,
               "-I" + os.path.join(ROOT, "include"), "-L" + libdir, "-ldeploy3d_b200", "-Wl,-rpath," + libdir,
               "-o", OUT]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("the TensorRT plugin shells do not compile:\n%s\n%s" % (" ".join(cmd), r.stderr))
    return OUT


_H = None


def harness():
    global _H
    if _H is None:
        h = ctypes.CDLL(build())
        vp, dp = ctypes.c_void_p, ctypes.POINTER(Desc)
        sig = {
            "t_num_creators": (ctypes.c_int, []),
            "t_creator_name": (ctypes.c_char_p, [ctypes.c_int]),
            "t_creator_version": (ctypes.c_char_p, [ctypes.c_int]),
            "t_creator_namespace": (ctypes.c_char_p, [ctypes.c_int]),
            "t_creator_refuses_fields": (ctypes.c_int, [ctypes.c_int]),
            "t_deserialize": (vp, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t]),
            "t_destroy": (None, [vp]),
            "t_clone": (vp, [vp]),
            "t_type": (ctypes.c_char_p, [vp]),
            "t_version": (ctypes.c_char_p, [vp]),
            "t_nb_outputs": (ctypes.c_int, [vp]),
            "t_serialization_size": (ctypes.c_size_t, [vp]),
            "t_serialize": (None, [vp, ctypes.c_char_p]),
            "t_output_dims": (ctypes.c_int, [vp, ctypes.c_int, dp, ctypes.c_int, dp]),
            "t_supports": (ctypes.c_int, [vp, ctypes.c_int, dp, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
            "t_workspace": (ctypes.c_size_t, [vp, dp, ctypes.c_int, dp, ctypes.c_int]),
            "t_configure_and_enqueue": (ctypes.c_int, [vp, dp, ctypes.c_int, dp, ctypes.c_int,
                                                        ctypes.POINTER(vp), ctypes.POINTER(vp), vp, vp]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(h, name)
            fn.restype, fn.argtypes = res, args
        _H = h
    return _H


def descs(items):
    """items: (dtype code, dims) pairs or objects with dtype / nb_dims / dims."""
    arr = (Desc * max(len(items), 1))()
    for i, it in enumerate(items):
        if isinstance(it, tuple):
            code, dims = it
            arr[i].dtype, arr[i].nb_dims = code, len(dims)
            for d, v in enumerate(dims):
                arr[i].dims[d] = int(v)
        else:
            arr[i].dtype, arr[i].nb_dims = it.dtype, it.nb_dims
            for d in range(it.nb_dims):
                arr[i].dims[d] = it.dims[d]
    return arr


class Shell:
    """A plugin created the way TensorRT creates it: creator.deserializePlugin(name, data_s)."""

    def __init__(self, name, data_s, ptr=None):
        self.h, self.name = harness(), name
        data_s = bytes(data_s)
        self.ptr = ptr if ptr is not None else self.h.t_deserialize(name.encode(), data_s, len(data_s))
        assert self.ptr, "no creator registered under %r" % name

    def close(self):
        if self.ptr:
            self.h.t_destroy(self.ptr)
            self.ptr = None

    def clone(self):
        return Shell(self.name, b"", ptr=self.h.t_clone(self.ptr))

    def serialize(self):
        n = self.h.t_serialization_size(self.ptr)
        buf = ctypes.create_string_buffer(max(n, 1))
        self.h.t_serialize(self.ptr, buf)
        return buf.raw[:n]

    def nb_outputs(self):
        return self.h.t_nb_outputs(self.ptr)

    def output_desc(self, index, in_descs):
        out = Desc()
        self.h.t_output_dims(self.ptr, index, descs(in_descs), len(in_descs), ctypes.byref(out))
        return out.dtype, [out.dims[d] for d in range(out.nb_dims)]

    def supports(self, pos, inout, n_in, n_out, non_linear=False):
        return bool(self.h.t_supports(self.ptr, pos, descs(inout), n_in, n_out, int(non_linear)))

    def workspace(self, in_descs, out_descs):
        return int(self.h.t_workspace(self.ptr, descs(in_descs), len(in_descs), descs(out_descs), len(out_descs)))

    def enqueue(self, inputs, outputs, workspace=None, stream=None):
        """configurePlugin + enqueue on torch CUDA tensors (zero-element tensors carry shapes only)."""
        import torch
        from deploy3d_b200.plugins import _desc_of
        din, dout = [_desc_of(t) for t in inputs], [_desc_of(t) for t in outputs]
        need = self.workspace(din, dout)
        if workspace is None and need:
            workspace = torch.empty(need, dtype=torch.uint8, device=inputs[0].device)
        vp = ctypes.c_void_p
        pin = (vp * len(inputs))(*[t.data_ptr() if t.numel() else None for t in inputs])
        pout = (vp * len(outputs))(*[t.data_ptr() if t.numel() else None for t in outputs])
        st = (stream or torch.cuda.current_stream(inputs[0].device)).cuda_stream
        return self.h.t_configure_and_enqueue(self.ptr, descs(din), len(din), descs(dout), len(dout), pin, pout,
                                              vp(workspace.data_ptr() if workspace is not None else 0), vp(st))
