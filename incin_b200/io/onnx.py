"""ONNX export and import for feed-forward models, with a self-contained protobuf codec (no ``onnx`` dependency).

Counterparts: the reference exports its traced graph to ONNX and imports ONNX / safetensors models into typed module
structs (``model!`` / ``import_model!`` in crates/incin-macros/src/lib.rs:88-341; the traced ``Graph`` of
crates/incin-core/src/tensor/tracing.rs is the export source).  Here :func:`export_module` walks a
``torch.nn.Sequential``-like module (Linear, activations, LayerNorm, Flatten, Dropout, Softmax) and writes a
``ModelProto`` with opset 17 nodes and raw-data initialisers; :func:`import_model` parses such a file back into an
:class:`OnnxGraph` that can be executed with torch ops or turned into an ``nn.Sequential`` again.

Only the protobuf fields this subset needs are encoded: ModelProto{ir_version=1, producer_name=2, graph=7,
opset_import=8}, GraphProto{node=1, name=2, initializer=5, input=11, output=12}, NodeProto{input=1, output=2, name=3,
op_type=4, attribute=5}, AttributeProto{name=1, f=2, i=3, ints=8, type=20}, TensorProto{dims=1, data_type=2, name=8,
raw_data=9}, ValueInfoProto{name=1, type=2}, TypeProto{tensor_type=1{elem_type=1, shape=2{dim=1{dim_value=1}}}}.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import torch
from torch import nn

from .limits import DEFAULT_LIMITS, ResourceLimits

FLOAT, INT64 = 1, 7
ATTR_FLOAT, ATTR_INT, ATTR_INTS = 1, 2, 7


# ---------------------------------------------------------------------------------------------------- protobuf wire
def _varint(n: int) -> bytes:
    if n < 0:
        n += 1 << 64
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _key(field_no: int, wire: int) -> bytes:
    return _varint((field_no << 3) | wire)


def _f_varint(field_no: int, v: int) -> bytes:
    return _key(field_no, 0) + _varint(v)


def _f_bytes(field_no: int, b: bytes) -> bytes:
    return _key(field_no, 2) + _varint(len(b)) + b


def _f_str(field_no: int, s: str) -> bytes:
    return _f_bytes(field_no, s.encode())


def _f_float(field_no: int, v: float) -> bytes:
    return _key(field_no, 5) + struct.pack("<f", v)


def _parse(buf: bytes) -> list[tuple[int, int, object]]:
    """One message level: [(field number, wire type, value)]; length-delimited values stay bytes."""
    out, i, n = [], 0, len(buf)
    while i < n:
        key, shift = 0, 0
        while True:
            b = buf[i]
            i += 1
            key |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                break
        field_no, wire = key >> 3, key & 7
        if wire == 0:
            v, shift = 0, 0
            while True:
                b = buf[i]
                i += 1
                v |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            out.append((field_no, wire, v))
        elif wire == 2:
            ln, shift = 0, 0
            while True:
                b = buf[i]
                i += 1
                ln |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            if i + ln > n:
                raise ValueError("truncated protobuf message")
            out.append((field_no, wire, bytes(buf[i:i + ln])))
            i += ln
        elif wire == 5:
            out.append((field_no, wire, struct.unpack_from("<f", buf, i)[0]))
            i += 4
        elif wire == 1:
            out.append((field_no, wire, struct.unpack_from("<d", buf, i)[0]))
            i += 8
        else:
            raise ValueError(f"unsupported protobuf wire type {wire}")
    return out


# ---------------------------------------------------------------------------------------------------- model objects
@dataclass
class OnnxNode:
    op_type: str
    inputs: list[str]
    outputs: list[str]
    attrs: dict = field(default_factory=dict)
    name: str = ""


@dataclass
class OnnxGraph:
    nodes: list[OnnxNode]
    initializers: dict[str, torch.Tensor]
    inputs: list[tuple[str, tuple[int, ...]]]
    outputs: list[tuple[str, tuple[int, ...]]]
    name: str = "incin_b200"

    def run(self, *feeds: torch.Tensor) -> list[torch.Tensor]:
        """Reference execution with torch ops (fp32 semantics of the ONNX operators in the exported subset)."""
        env = dict(self.initializers)
        for (name, _), t in zip(self.inputs, feeds):
            env[name] = t
        for n in self.nodes:
            x = [env[i] for i in n.inputs]
            a = n.attrs
            if n.op_type == "Gemm":
                w = x[1].t() if a.get("transB", 0) else x[1]
                y = a.get("alpha", 1.0) * (x[0] @ w)
                if len(x) > 2:
                    y = y + a.get("beta", 1.0) * x[2]
            elif n.op_type == "MatMul":
                y = x[0] @ x[1]
            elif n.op_type == "Add":
                y = x[0] + x[1]
            elif n.op_type == "Relu":
                y = torch.relu(x[0])
            elif n.op_type == "Sigmoid":
                y = torch.sigmoid(x[0])
            elif n.op_type == "Tanh":
                y = torch.tanh(x[0])
            elif n.op_type == "Gelu":
                y = nn.functional.gelu(x[0])
            elif n.op_type == "Softmax":
                y = torch.softmax(x[0], a.get("axis", -1))
            elif n.op_type == "Flatten":
                y = x[0].flatten(a.get("axis", 1))
            elif n.op_type == "Identity":
                y = x[0]
            elif n.op_type == "LayerNormalization":
                y = nn.functional.layer_norm(x[0], x[1].shape, x[1], x[2] if len(x) > 2 else None, a.get("epsilon", 1e-5))
            else:
                raise NotImplementedError(f"ONNX operator {n.op_type}")
            env[n.outputs[0]] = y
        return [env[name] for name, _ in self.outputs]

    def to_module(self) -> nn.Sequential:
        """Rebuild a sequential torch module (every node must feed the next one)."""
        layers: list[nn.Module] = []
        for n in self.nodes:
            a = n.attrs
            if n.op_type == "Gemm":
                w = self.initializers[n.inputs[1]]
                w = w if a.get("transB", 0) else w.t()
                lin = nn.Linear(w.shape[1], w.shape[0], bias=len(n.inputs) > 2)
                with torch.no_grad():
                    lin.weight.copy_(w)
                    if len(n.inputs) > 2:
                        lin.bias.copy_(self.initializers[n.inputs[2]])
                layers.append(lin)
            elif n.op_type in ("Relu", "Sigmoid", "Tanh"):
                layers.append({"Relu": nn.ReLU, "Sigmoid": nn.Sigmoid, "Tanh": nn.Tanh}[n.op_type]())
            elif n.op_type == "Gelu":
                layers.append(nn.GELU())
            elif n.op_type == "Softmax":
                layers.append(nn.Softmax(a.get("axis", -1)))
            elif n.op_type == "Flatten":
                layers.append(nn.Flatten(a.get("axis", 1)))
            elif n.op_type == "Identity":
                layers.append(nn.Identity())
            elif n.op_type == "LayerNormalization":
                g = self.initializers[n.inputs[1]]
                ln = nn.LayerNorm(tuple(g.shape), eps=a.get("epsilon", 1e-5))
                with torch.no_grad():
                    ln.weight.copy_(g)
                    if len(n.inputs) > 2:
                        ln.bias.copy_(self.initializers[n.inputs[2]])
                layers.append(ln)
            else:
                raise NotImplementedError(f"ONNX operator {n.op_type}")
        return nn.Sequential(*layers)


# ---------------------------------------------------------------------------------------------------- export
def _tensor_proto(name: str, t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.is_floating_point():
        t, code = t.float(), FLOAT
    else:
        t, code = t.long(), INT64
    body = b"".join(_f_varint(1, d) for d in t.shape) + _f_varint(2, code) + _f_str(8, name)
    return body + _f_bytes(9, t.numpy().tobytes())


def _value_info(name: str, shape) -> bytes:
    dims = b"".join(_f_bytes(1, _f_varint(1, d)) for d in shape)
    tensor_type = _f_varint(1, FLOAT) + _f_bytes(2, dims)
    return _f_str(1, name) + _f_bytes(2, _f_bytes(1, tensor_type))


def _attr(name: str, v) -> bytes:
    if isinstance(v, float):
        return _f_str(1, name) + _f_float(2, v) + _f_varint(20, ATTR_FLOAT)
    if isinstance(v, int):
        return _f_str(1, name) + _f_varint(3, v) + _f_varint(20, ATTR_INT)
    return _f_str(1, name) + b"".join(_f_varint(8, int(i)) for i in v) + _f_varint(20, ATTR_INTS)


def _node_proto(n: OnnxNode) -> bytes:
    return (b"".join(_f_str(1, i) for i in n.inputs) + b"".join(_f_str(2, o) for o in n.outputs) + _f_str(3, n.name) +
            _f_str(4, n.op_type) + b"".join(_f_bytes(5, _attr(k, v)) for k, v in n.attrs.items()))


def graph_of_module(module: nn.Module, input_shape) -> OnnxGraph:
    """Lower a sequential module to ONNX nodes (shapes are propagated on meta tensors)."""
    layers = list(module.children()) if not isinstance(module, (nn.Linear, nn.LayerNorm)) else [module]
    nodes, inits = [], {}
    cur, shape = "input", tuple(input_shape)
    probe = torch.empty(shape, device="meta")
    for i, layer in enumerate(layers):
        out = f"t{i}"
        kind = type(layer).__name__
        if isinstance(layer, nn.Linear) or kind == "Linear":
            inits[f"l{i}.weight"] = layer.weight
            ins = [cur, f"l{i}.weight"]
            if layer.bias is not None:
                inits[f"l{i}.bias"] = layer.bias
                ins.append(f"l{i}.bias")
            nodes.append(OnnxNode("Gemm", ins, [out], {"transB": 1, "alpha": 1.0, "beta": 1.0}, f"gemm{i}"))
            probe = torch.empty(probe.shape[:-1] + (layer.weight.shape[0],), device="meta")
        elif isinstance(layer, nn.LayerNorm) or kind == "LayerNorm":
            inits[f"l{i}.weight"] = layer.weight
            ins = [cur, f"l{i}.weight"]
            if getattr(layer, "bias", None) is not None:
                inits[f"l{i}.bias"] = layer.bias
                ins.append(f"l{i}.bias")
            nodes.append(OnnxNode("LayerNormalization", ins, [out], {"axis": -1, "epsilon": float(layer.eps)}, f"ln{i}"))
        elif kind in ("ReLU", "Sigmoid", "Tanh"):
            nodes.append(OnnxNode({"ReLU": "Relu"}.get(kind, kind), [cur], [out], {}, f"act{i}"))
        elif kind in ("GELU",):
            nodes.append(OnnxNode("Gelu", [cur], [out], {}, f"act{i}"))
        elif kind == "Softmax":
            nodes.append(OnnxNode("Softmax", [cur], [out], {"axis": int(getattr(layer, "dim", -1) or -1)}, f"softmax{i}"))
        elif kind == "Flatten":
            probe = probe.flatten(1)
            nodes.append(OnnxNode("Flatten", [cur], [out], {"axis": 1}, f"flatten{i}"))
        elif kind in ("Dropout", "Identity"):
            nodes.append(OnnxNode("Identity", [cur], [out], {}, f"id{i}"))      # inference graph: dropout is the identity
        else:
            raise NotImplementedError(f"no ONNX lowering for layer {kind}")
        cur = out
    return OnnxGraph(nodes, {k: v.detach().float().cpu() for k, v in inits.items()}, [("input", shape)],
                     [(cur, tuple(probe.shape))])


def write_onnx(path, g: OnnxGraph) -> None:
    graph = (b"".join(_f_bytes(1, _node_proto(n)) for n in g.nodes) + _f_str(2, g.name) +
             b"".join(_f_bytes(5, _tensor_proto(k, v)) for k, v in g.initializers.items()) +
             b"".join(_f_bytes(11, _value_info(n, s)) for n, s in g.inputs) +
             b"".join(_f_bytes(12, _value_info(n, s)) for n, s in g.outputs))
    model = (_f_varint(1, 8) + _f_str(2, "incin_b200") + _f_bytes(7, graph) +
             _f_bytes(8, _f_str(1, "") + _f_varint(2, 17)))
    with open(path, "wb") as f:
        f.write(model)


def export_module(module: nn.Module, input_shape, path) -> OnnxGraph:
    g = graph_of_module(module, input_shape)
    write_onnx(path, g)
    return g


# ---------------------------------------------------------------------------------------------------- import
def _read_tensor(buf: bytes) -> tuple[str, torch.Tensor]:
    dims, code, name, raw = [], FLOAT, "", b""
    for f, w, v in _parse(buf):
        if f == 1 and w == 0:
            dims.append(v)
        elif f == 1 and w == 2:          # packed dims
            dims += _unpack_varints(v)
        elif f == 2:
            code = v
        elif f == 8:
            name = v.decode()
        elif f == 9:
            raw = v
    dtype = {FLOAT: torch.float32, INT64: torch.int64}.get(code)
    if dtype is None:
        raise NotImplementedError(f"ONNX tensor data type {code}")
    t = torch.frombuffer(bytearray(raw), dtype=dtype).reshape(dims) if raw else torch.zeros(dims, dtype=dtype)
    return name, t.clone()


def _unpack_varints(b: bytes) -> list[int]:
    out, i = [], 0
    while i < len(b):
        v, shift = 0, 0
        while True:
            c = b[i]
            i += 1
            v |= (c & 0x7F) << shift
            shift += 7
            if not c & 0x80:
                break
        out.append(v)
    return out


def _read_value_info(buf: bytes) -> tuple[str, tuple[int, ...]]:
    name, shape = "", []
    for f, _, v in _parse(buf):
        if f == 1:
            name = v.decode()
        elif f == 2:
            for f2, _, v2 in _parse(v):
                if f2 == 1:
                    for f3, _, v3 in _parse(v2):
                        if f3 == 2:
                            for f4, _, v4 in _parse(v3):
                                if f4 == 1:
                                    dv = [x for fx, _, x in _parse(v4) if fx == 1]
                                    shape.append(dv[0] if dv else -1)
    return name, tuple(shape)


def _read_node(buf: bytes) -> OnnxNode:
    n = OnnxNode("", [], [])
    for f, _, v in _parse(buf):
        if f == 1:
            n.inputs.append(v.decode())
        elif f == 2:
            n.outputs.append(v.decode())
        elif f == 3:
            n.name = v.decode()
        elif f == 4:
            n.op_type = v.decode()
        elif f == 5:
            name, val, ints = "", None, []
            for fa, wa, va in _parse(v):
                if fa == 1:
                    name = va.decode()
                elif fa == 2:
                    val = float(va)
                elif fa == 3:
                    val = va - (1 << 64) if va >= (1 << 63) else va
                elif fa == 8:
                    ints += _unpack_varints(va) if wa == 2 else [va]
            n.attrs[name] = ints if ints else val
    return n


def import_model(path, limits: ResourceLimits = DEFAULT_LIMITS) -> OnnxGraph:
    import os
    limits.check("file size", os.path.getsize(path), limits.max_file_bytes)
    raw = open(path, "rb").read()
    graph_buf = None
    for f, _, v in _parse(raw):
        if f == 7:
            graph_buf = v
    if graph_buf is None:
        raise ValueError("not an ONNX model: no graph")
    g = OnnxGraph([], {}, [], [])
    for f, _, v in _parse(graph_buf):
        if f == 1:
            g.nodes.append(_read_node(v))
        elif f == 2:
            g.name = v.decode()
        elif f == 5:
            name, t = _read_tensor(v)
            g.initializers[name] = t
        elif f == 11:
            g.inputs.append(_read_value_info(v))
        elif f == 12:
            g.outputs.append(_read_value_info(v))
    limits.check("graph nodes", len(g.nodes), limits.max_graph_nodes)
    limits.check("tensor count", len(g.initializers), limits.max_tensor_count)
    g.inputs = [(n, s) for n, s in g.inputs if n not in g.initializers]
    return g


export_onnx, import_onnx = export_module, import_model      # the exporter / importer under the reference's names
