"""Write (and read back) TensorFlow frozen graphs, the model format ``cuBERT_open`` takes.

A frozen BERT graph is a ``GraphDef`` whose weights are ``Const`` nodes carrying a
``value`` attribute with a ``TensorProto``. Only the fields the reference's loader reads
are produced (src/cuBERT/tensorflow/Graph.cpp:28-79; field numbers from
tensorflow/core/framework/{graph,node_def,attr_value,tensor,tensor_shape,types}.proto):

    GraphDef.node = 1 -> NodeDef{name = 1, op = 2, attr = 5 (map entry key = 1, value = 2)}
    AttrValue{type = 6, tensor = 8}
    TensorProto{dtype = 1, tensor_shape = 2 -> dim = 2 -> size = 1, tensor_content = 4}
    DT_FLOAT = 1, DT_HALF = 19

The wire format is encoded by hand; no protobuf package is needed. Used by the tests and
the benchmark to put seeded random weights into a file the C API can open.
"""
import numpy as np

DT_FLOAT = 1
DT_HALF = 19


def _varint(n):
    out = bytearray()
    n &= (1 << 64) - 1
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field, wire_type):
    return _varint((field << 3) | wire_type)


def _len_delimited(field, payload):
    return _key(field, 2) + _varint(len(payload)) + payload


def _tensor_proto(arr, declared_shape=None):
    arr = np.ascontiguousarray(arr)
    if arr.dtype == np.float32:
        dtype = DT_FLOAT
    elif arr.dtype == np.float16:
        dtype = DT_HALF
    else:
        raise TypeError("only float32 and float16 tensors are written, got %s" % arr.dtype)
    dims = arr.shape if declared_shape is None else declared_shape
    shape = b"".join(_len_delimited(2, _key(1, 0) + _varint(int(d))) for d in dims)
    return dtype, (_key(1, 0) + _varint(dtype) + _len_delimited(2, shape) +
                   _len_delimited(4, arr.tobytes()))


def _const_node(name, arr, declared_shape=None):
    dtype, tensor = _tensor_proto(arr, declared_shape)
    attr_dtype = _len_delimited(1, b"dtype") + _len_delimited(2, _key(6, 0) + _varint(dtype))
    attr_value = _len_delimited(1, b"value") + _len_delimited(2, _len_delimited(8, tensor))
    return (_len_delimited(1, name.encode()) + _len_delimited(2, b"Const") +
            _len_delimited(5, attr_dtype) + _len_delimited(5, attr_value))


def write_frozen_graph(path, var, extra_nodes=(), declared_shapes=None):
    """var: {TensorFlow variable name: float32/float16 array}. extra_nodes: names of
    weight-less nodes to interleave (a real graph has many; the loader must skip them).
    declared_shapes: {name: dims} written as the tensor's shape in place of the array's own
    (for tests of files whose shape and content disagree)."""
    declared_shapes = declared_shapes or {}
    with open(path, "wb") as f:
        for name in extra_nodes:
            node = _len_delimited(1, name.encode()) + _len_delimited(2, b"Identity") + \
                _len_delimited(3, b"some/input")
            f.write(_len_delimited(1, node))
        for name, arr in var.items():
            f.write(_len_delimited(1, _const_node(name, arr, declared_shapes.get(name))))
        # GraphDef.versions = 4 { producer = 1 }: an unknown-to-the-loader field at the end
        f.write(_len_delimited(4, _key(1, 0) + _varint(27)))


# ------------------------------------------------------------------ reader (for round-trip tests)

def _read_varint(buf, pos):
    shift = 0
    val = 0
    while True:
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7


def _fields(buf):
    pos = 0
    end = len(buf)
    while pos < end:
        key, pos = _read_varint(buf, pos)
        field, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _read_varint(buf, pos)
        elif wt == 1:
            val, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            n, pos = _read_varint(buf, pos)
            val, pos = buf[pos:pos + n], pos + n
        elif wt == 5:
            val, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError("unsupported wire type %d" % wt)
        yield field, wt, val


def read_frozen_graph(path):
    """{name: array} of every float32/float16 'value' tensor, as the C++ loader sees them."""
    with open(path, "rb") as f:
        buf = memoryview(f.read())
    out = {}
    for field, wt, node in _fields(buf):
        if field != 1 or wt != 2:
            continue
        name, tensor = None, None
        for nf, nwt, nval in _fields(node):
            if nf == 1 and nwt == 2:
                name = bytes(nval).decode()
            elif nf == 5 and nwt == 2:
                key, val = None, None
                for ef, ewt, eval_ in _fields(nval):
                    if ef == 1:
                        key = bytes(eval_)
                    elif ef == 2:
                        val = eval_
                if key == b"value" and val is not None:
                    for af, awt, aval in _fields(val):
                        if af == 8 and awt == 2:
                            tensor = aval
        if tensor is None:
            continue
        dtype, dims, content = 0, [], b""
        for tf, twt, tval in _fields(tensor):
            if tf == 1 and twt == 0:
                dtype = tval
            elif tf == 2 and twt == 2:
                for sf, swt, sval in _fields(tval):
                    if sf == 2 and swt == 2:
                        size = 0
                        for df, dwt, dval in _fields(sval):
                            if df == 1 and dwt == 0:
                                size = dval
                        dims.append(size)
            elif tf == 4 and twt == 2:
                content = bytes(tval)
        if dtype == DT_FLOAT:
            out[name] = np.frombuffer(content, np.float32).reshape(dims)
        elif dtype == DT_HALF:
            out[name] = np.frombuffer(content, np.float16).reshape(dims)
    return out
