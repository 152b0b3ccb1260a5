"""Drives the IPluginV3 objects of libbert_b200_plugin.so through the C harness (csrc/plugin/harness.cpp), i.e.
through their real virtual interfaces, without TensorRT. The ctypes structs mirror the POD types of the public
TensorRT headers (PluginField, PluginFieldCollection, Dims64, PluginTensorDesc, DynamicPluginTensorDesc).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import _lib  # noqa: F401  (libbert_b200.so must be loaded first: the plugin library links against it)

PLUGIN_LIB_PATH = Path(__file__).resolve().parent / "libbert_b200_plugin.so"
if not PLUGIN_LIB_PATH.exists():
    raise ImportError(f"{PLUGIN_LIB_PATH} is missing: build it with `python tensorrt_b200/csrc/build.py` "
                      "(needs the public TensorRT headers, e.g. TENSORRT_INCLUDE_DIR)")
plib = C.CDLL(str(PLUGIN_LIB_PATH), mode=C.RTLD_GLOBAL)

# nvinfer1::DataType, TensorFormat, PluginFieldType, TensorRTPhase
FLOAT, HALF, INT8, INT32 = 0, 1, 2, 3
LINEAR, CHW4, CHW32 = 0, 3, 5
F_FLOAT16, F_FLOAT32, F_INT32, F_UNKNOWN = 0, 1, 5, 8
BUILD, RUNTIME = 0, 1


class PluginField(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("type", C.c_int32), ("length", C.c_int32)]


class PluginFieldCollection(C.Structure):
    _fields_ = [("nbFields", C.c_int32), ("fields", C.POINTER(PluginField))]


class Dims(C.Structure):
    _fields_ = [("nbDims", C.c_int32), ("d", C.c_int64 * 8)]


class PluginTensorDesc(C.Structure):
    _fields_ = [("dims", Dims), ("type", C.c_int32), ("format", C.c_int32), ("scale", C.c_float)]


class DynamicPluginTensorDesc(C.Structure):
    _fields_ = [("desc", PluginTensorDesc), ("min", Dims), ("max", Dims), ("opt", Dims)]


plib.bert_b200_harness_create.restype = C.c_void_p
plib.bert_b200_harness_create.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(PluginFieldCollection), C.c_int32]
plib.bert_b200_harness_clone.restype = C.c_void_p
plib.bert_b200_harness_clone.argtypes = [C.c_void_p]
plib.bert_b200_harness_attach.restype = C.c_void_p
plib.bert_b200_harness_attach.argtypes = [C.c_void_p]
plib.bert_b200_harness_destroy.argtypes = [C.c_void_p]
plib.bert_b200_harness_serialize.restype = C.POINTER(PluginFieldCollection)
plib.bert_b200_harness_serialize.argtypes = [C.c_void_p]
plib.bert_b200_harness_workspace_size.restype = C.c_int64
plib.bert_b200_harness_creator_field_name.restype = C.c_char_p
for _n in ("nb_outputs", "supports_format", "output_shapes", "output_types", "configure", "workspace_size",
           "on_shape_change", "enqueue", "core_info"):
    getattr(plib, "bert_b200_harness_" + _n).argtypes = None


def make_dims(shape) -> Dims:
    d = Dims()
    d.nbDims = len(shape)
    for i, v in enumerate(shape):
        d.d[i] = int(v)
    return d


def make_desc(shape, dtype, fmt=LINEAR, scale=1.0) -> PluginTensorDesc:
    return PluginTensorDesc(make_dims(shape), dtype, fmt, scale)


def make_dyn(shape, dtype, fmt=LINEAR, scale=1.0) -> DynamicPluginTensorDesc:
    dims = make_dims(shape)
    return DynamicPluginTensorDesc(make_desc(shape, dtype, fmt, scale), dims, dims, dims)


class FieldCollection:
    """Builds a PluginFieldCollection from (name, value) pairs; value is an int, a float or a numpy array
    (float32 / float16 / int32). Keeps the backing memory alive."""

    def __init__(self, items):
        self._keep = []
        fields = []
        for name, value in items:
            if isinstance(value, (bool, int, np.integer)):
                arr, ftype = np.array([value], dtype=np.int32), F_INT32
            elif isinstance(value, (float, np.floating)):
                arr, ftype = np.array([value], dtype=np.float32), F_FLOAT32
            else:
                arr = np.ascontiguousarray(value)
                ftype = {np.dtype(np.float32): F_FLOAT32, np.dtype(np.float16): F_FLOAT16,
                         np.dtype(np.int32): F_INT32}.get(arr.dtype, F_UNKNOWN)
            self._keep.append(arr)
            bname = name.encode()
            self._keep.append(bname)
            fields.append(PluginField(bname, arr.ctypes.data, ftype, arr.size))
        self._array = (PluginField * len(fields))(*fields)
        self.fc = PluginFieldCollection(len(fields), self._array)


def read_fields(fc_ptr) -> dict:
    """PluginFieldCollection* -> {name: numpy array copy} (what an engine file would store)."""
    out = {}
    fc = fc_ptr.contents
    for i in range(fc.nbFields):
        f = fc.fields[i]
        dt = {F_FLOAT16: np.float16, F_FLOAT32: np.float32, F_INT32: np.int32}.get(f.type, np.uint8)
        n = f.length
        buf = (C.c_uint8 * (n * np.dtype(dt).itemsize)).from_address(f.data) if f.data and n else b""
        out[f.name.decode()] = np.frombuffer(bytes(buf), dtype=dt).copy()
    return out


def creators():
    """[(name, version, namespace, [field names])] of every creator getCreators() returns."""
    res = []
    for i in range(plib.bert_b200_harness_num_creators()):
        name, ver, ns, nb = C.c_char_p(), C.c_char_p(), C.c_char_p(), C.c_int32()
        plib.bert_b200_harness_creator_info(i, C.byref(name), C.byref(ver), C.byref(ns), C.byref(nb))
        fields = [plib.bert_b200_harness_creator_field_name(i, f).decode() for f in range(nb.value)]
        res.append((name.value.decode(), ver.value.decode(), ns.value.decode(), fields))
    return res


class Plugin:
    def __init__(self, name, version, items, phase=BUILD, handle=None):
        if handle is None:
            self._fc = FieldCollection(items)
            handle = plib.bert_b200_harness_create(name.encode(), version.encode(), C.byref(self._fc.fc), phase)
        self.h = handle  # None when the creator refused the fields (createPlugin returned nullptr)

    @property
    def ok(self):
        return bool(self.h)

    def close(self):
        if self.h:
            plib.bert_b200_harness_destroy(C.c_void_p(self.h))
            self.h = None

    def clone(self):
        return Plugin(None, None, None, handle=plib.bert_b200_harness_clone(C.c_void_p(self.h)))

    def attach(self):
        return Plugin(None, None, None, handle=plib.bert_b200_harness_attach(C.c_void_p(self.h)))

    def core_info(self):
        name, ver, ns = C.c_char_p(), C.c_char_p(), C.c_char_p()
        plib.bert_b200_harness_core_info(C.c_void_p(self.h), C.byref(name), C.byref(ver), C.byref(ns))
        return name.value.decode(), ver.value.decode(), ns.value.decode()

    def nb_outputs(self):
        return plib.bert_b200_harness_nb_outputs(C.c_void_p(self.h))

    def supports(self, pos, descs, nb_in, nb_out):
        arr = (DynamicPluginTensorDesc * len(descs))(*descs)
        return plib.bert_b200_harness_supports_format(C.c_void_p(self.h), pos, arr, nb_in, nb_out) == 1

    def output_shapes(self, in_shapes, nb_out):
        ins = (Dims * len(in_shapes))(*[make_dims(s) for s in in_shapes])
        outs = (Dims * nb_out)()
        st = plib.bert_b200_harness_output_shapes(C.c_void_p(self.h), ins, len(in_shapes), outs, nb_out)
        if st != 0:
            return None
        return [tuple(o.d[i] for i in range(o.nbDims)) for o in outs]

    def output_types(self, in_types, nb_out):
        it = (C.c_int32 * len(in_types))(*in_types)
        ot = (C.c_int32 * nb_out)()
        st = plib.bert_b200_harness_output_types(C.c_void_p(self.h), ot, nb_out, it, len(in_types))
        return None if st != 0 else list(ot)

    def configure(self, ins, outs):
        a = (DynamicPluginTensorDesc * len(ins))(*ins)
        b = (DynamicPluginTensorDesc * len(outs))(*outs)
        return plib.bert_b200_harness_configure(C.c_void_p(self.h), a, len(ins), b, len(outs))

    def workspace_size(self, ins, outs):
        a = (DynamicPluginTensorDesc * len(ins))(*ins)
        b = (DynamicPluginTensorDesc * len(outs))(*outs)
        return plib.bert_b200_harness_workspace_size(C.c_void_p(self.h), a, len(ins), b, len(outs))

    def on_shape_change(self, ins, outs):
        a = (PluginTensorDesc * len(ins))(*ins)
        b = (PluginTensorDesc * len(outs))(*outs)
        return plib.bert_b200_harness_on_shape_change(C.c_void_p(self.h), a, len(ins), b, len(outs))

    def enqueue(self, in_descs, out_descs, in_ptrs, out_ptrs, workspace=None, stream=None):
        a = (PluginTensorDesc * len(in_descs))(*in_descs)
        b = (PluginTensorDesc * len(out_descs))(*out_descs)
        ip = (C.c_void_p * len(in_ptrs))(*in_ptrs)
        op = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        return plib.bert_b200_harness_enqueue(C.c_void_p(self.h), a, b, ip, op, C.c_void_p(workspace or 0),
                                              C.c_void_p(stream or 0))

    def serialize(self) -> dict:
        return read_fields(plib.bert_b200_harness_serialize(C.c_void_p(self.h)))


# ---- legacy IPluginV2DynamicExt objects -------------------------------------------------------------------------
for _n in ("legacy_create", "legacy_deserialize", "legacy_clone"):
    getattr(plib, "bert_b200_harness_" + _n).restype = C.c_void_p
plib.bert_b200_harness_legacy_create.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(PluginFieldCollection)]
plib.bert_b200_harness_legacy_deserialize.argtypes = [C.c_char_p, C.c_char_p, C.c_void_p, C.c_int64]
plib.bert_b200_harness_legacy_clone.argtypes = [C.c_void_p]
plib.bert_b200_harness_legacy_destroy.argtypes = [C.c_void_p]
plib.bert_b200_harness_legacy_workspace_size.restype = C.c_int64
plib.bert_b200_harness_legacy_serialization_size.restype = C.c_int64
plib.bert_b200_harness_legacy_serialization_size.argtypes = [C.c_void_p]


def legacy_creators():
    """[(name, version)] of the IPluginCreator (legacy plugin) entries getCreators() returns."""
    res = []
    for i, (name, ver, _, _) in enumerate(creators()):
        if plib.bert_b200_harness_creator_is_legacy(i) == 1:
            res.append((name, ver))
    return res


class LegacyPlugin:
    """An IPluginV2DynamicExt object of a legacy plugin version, created from fields or from a serialised buffer."""

    def __init__(self, name, version, items=None, serialized: bytes | None = None, handle=None):
        self.name, self.version = name, version
        if handle is None:
            if serialized is not None:
                self._buf = C.create_string_buffer(serialized, len(serialized))
                handle = plib.bert_b200_harness_legacy_deserialize(name.encode(), version.encode(), self._buf, len(serialized))
            else:
                self._fc = FieldCollection(items)
                handle = plib.bert_b200_harness_legacy_create(name.encode(), version.encode(), C.byref(self._fc.fc))
        self.h = handle

    @property
    def ok(self):
        return bool(self.h)

    def close(self):
        if self.h:
            plib.bert_b200_harness_legacy_destroy(C.c_void_p(self.h))
            self.h = None

    def clone(self):
        return LegacyPlugin(self.name, self.version, handle=plib.bert_b200_harness_legacy_clone(C.c_void_p(self.h)))

    def info(self):
        t, ver, ns = C.c_char_p(), C.c_char_p(), C.c_char_p()
        plib.bert_b200_harness_legacy_info(C.c_void_p(self.h), C.byref(t), C.byref(ver), C.byref(ns))
        return t.value.decode(), ver.value.decode(), ns.value.decode()

    def nb_outputs(self):
        return plib.bert_b200_harness_legacy_nb_outputs(C.c_void_p(self.h))

    def supports(self, pos, descs, nb_in, nb_out):
        arr = (PluginTensorDesc * len(descs))(*descs)
        return plib.bert_b200_harness_legacy_supports_format(C.c_void_p(self.h), pos, arr, nb_in, nb_out) == 1

    def output_dims(self, index, in_shapes):
        ins = (Dims * len(in_shapes))(*[make_dims(s) for s in in_shapes])
        out = Dims()
        st = plib.bert_b200_harness_legacy_output_dims(C.c_void_p(self.h), index, ins, len(in_shapes), C.byref(out))
        return None if st != 0 else tuple(out.d[i] for i in range(out.nbDims))

    def output_type(self, index, in_types):
        it = (C.c_int32 * len(in_types))(*in_types)
        return plib.bert_b200_harness_legacy_output_type(C.c_void_p(self.h), index, it, len(in_types))

    def configure(self, ins, outs):
        a = (DynamicPluginTensorDesc * len(ins))(*ins)
        b = (DynamicPluginTensorDesc * len(outs))(*outs)
        return plib.bert_b200_harness_legacy_configure(C.c_void_p(self.h), a, len(ins), b, len(outs))

    def workspace_size(self, ins, outs):
        a = (PluginTensorDesc * len(ins))(*ins)
        b = (PluginTensorDesc * len(outs))(*outs)
        return plib.bert_b200_harness_legacy_workspace_size(C.c_void_p(self.h), a, len(ins), b, len(outs))

    def enqueue(self, in_descs, out_descs, in_ptrs, out_ptrs, workspace=None, stream=None):
        a = (PluginTensorDesc * len(in_descs))(*in_descs)
        b = (PluginTensorDesc * len(out_descs))(*out_descs)
        ip = (C.c_void_p * len(in_ptrs))(*in_ptrs)
        op = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        return plib.bert_b200_harness_legacy_enqueue(C.c_void_p(self.h), a, b, ip, op, C.c_void_p(workspace or 0),
                                                     C.c_void_p(stream or 0))

    def serialize(self) -> bytes:
        n = plib.bert_b200_harness_legacy_serialization_size(C.c_void_p(self.h))
        buf = C.create_string_buffer(int(n))
        st = plib.bert_b200_harness_legacy_serialize(C.c_void_p(self.h), buf)
        assert st == 0
        return bytes(buf.raw)
