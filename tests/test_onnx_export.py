"""ONNX export of the decoder with KV-cache ports (dl_onnx_save_decoder; extensions/onnx/src/decoder.cpp:53-118 of the
reference).  The files this library writes must equal, byte for byte, the files the reference's own exporter wrote for the
same seeded weights: tests/golden/*.onnx (made by tests/golden/make_golden.py from the reference build) and, where the
reference build is present, files written on the spot for other shapes.  A small protobuf reader checks the structure
independently of the byte comparison: port names and shapes, one Attention node per layer, interleaved RoPE."""
import os
import sys

import numpy as np
import pytest

import ctorch_b200 as B
import oracle
from ctorch_b200 import workloads as W

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from cases import archive_cases  # noqa: E402


def fields(data: bytes):
    """(field number, wire type, value) triples of one protobuf message; length-delimited values stay bytes."""
    at, out = 0, []

    def varint():
        nonlocal at
        shift = value = 0
        while True:
            byte = data[at]
            at += 1
            value |= (byte & 0x7F) << shift
            shift += 7
            if byte < 0x80:
                return value

    while at < len(data):
        key = varint()
        number, wire = key >> 3, key & 7
        if wire == 0:
            out.append((number, wire, varint()))
        elif wire == 2:
            size = varint()
            out.append((number, wire, data[at:at + size]))
            at += size
        elif wire == 5:
            out.append((number, wire, data[at:at + 4]))
            at += 4
        else:
            raise AssertionError(f"unexpected wire type {wire}")
    return out


def port(info: bytes):
    """(name, element type, dims) of a ValueInfoProto; dims are ints or symbolic names."""
    parts = dict((n, v) for n, _, v in fields(info))
    tensor = dict((n, v) for n, _, v in fields(dict((n, v) for n, _, v in fields(parts[2]))[1]))
    dims = []
    for _, _, dim in fields(tensor[2]):
        (number, _, value), = fields(dim)
        dims.append(value if number == 1 else value.decode())
    return parts[1].decode(), tensor[1], dims


def graph_of(path):
    model = fields(open(path, "rb").read())
    assert [v for n, _, v in model if n == 1] == [12] and [v for n, _, v in model if n == 2] == [b"Ctorch"]
    (opset,) = [v for n, _, v in model if n == 8]
    assert fields(opset) == [(2, 0, 24)]
    (graph,) = [v for n, _, v in model if n == 7]
    return fields(graph)


@pytest.mark.parametrize("name", sorted(archive_cases()))
@pytest.mark.parametrize("with_head", [False, True])
def test_export_equals_the_reference_written_file(name, with_head, tmp_path):
    spec = archive_cases()[name]
    model = B.DecoderModel(spec, W.make_weights(spec, seed=77), device=None)     # modules on the host: the export runs no kernel
    path = str(tmp_path / "mine.onnx")
    model.save_onnx(path, with_head)
    golden = os.path.join(HERE, "golden", name + ("_lm.onnx" if with_head else "_decoder.onnx"))
    assert open(path, "rb").read() == open(golden, "rb").read()
    # structure, read back without the reference
    graph = graph_of(path)
    inputs = [port(v) for n, _, v in graph if n == 11]
    outputs = [port(v) for n, _, v in graph if n == 12]
    hd, kv = spec["d_model"] // spec["heads"], spec["kv_heads"]
    first_in = ("input_ids", 7, ["batch", "tokens"]) if with_head else ("features", 1, ["batch", "tokens", spec["d_model"]])
    first_out = ("logits", 1, ["batch", "tokens", spec["vocab"]]) if with_head else ("hidden_states", 1, ["batch", "tokens", spec["d_model"]])
    assert inputs[0] == first_in and outputs[0] == first_out
    for i in range(spec["layers"]):
        assert inputs[1 + 2 * i] == (f"past_key_{i}", 1, ["batch", kv, "past", hd])
        assert inputs[2 + 2 * i] == (f"past_value_{i}", 1, ["batch", kv, "past", hd])
        assert outputs[1 + 2 * i] == (f"present_key_{i}", 1, ["batch", kv, "total", hd])
        assert outputs[2 + 2 * i] == (f"present_value_{i}", 1, ["batch", kv, "total", hd])
    nodes = [fields(v) for n, _, v in graph if n == 1]
    kinds = [dict((n, v) for n, _, v in node if n == 4)[4].decode() for node in nodes]
    assert kinds.count("Attention") == spec["layers"] and kinds.count("RotaryEmbedding") == 2 * spec["layers"]
    assert kinds.count("RMSNormalization") == 2 * spec["layers"] + 1 and kinds[-1] == "Identity"
    for node, kind in zip(nodes, kinds):
        attributes = [dict((n, v) for n, _, v in fields(v)) for n, _, v in node if n == 5]
        if kind == "RotaryEmbedding":
            assert attributes == [{1: b"interleaved", 20: 2, 3: 1}]        # adjacent pairs, as dl::rotary_embedding rotates them
        if kind == "Attention":
            assert attributes == [{1: b"is_causal", 20: 2, 3: 1}]
            assert [v.decode() for n, _, v in node if n == 1][3:] == ["", f"past_key_{kinds[:nodes.index(node)].count('Attention')}",
                                                                     f"past_value_{kinds[:nodes.index(node)].count('Attention')}"]
    # the tied table is one initializer: vocab x d_model floats appear once
    table_bytes = spec["vocab"] * spec["d_model"] * 4
    assert sum(1 for n, _, v in graph if n == 5 and len(dict((a, b) for a, _, b in fields(v))[9]) == table_bytes) == (1 if with_head else 0)


@pytest.mark.skipif(not oracle.have_ref(), reason="needs the reference build (oracle/_ref)")
@pytest.mark.parametrize("dtype,tied", [("f32", True), ("bf16", False)])
def test_export_equals_a_fresh_reference_export(dtype, tied, tmp_path):
    """Other shapes than the committed fixtures (three layers, grouped heads, an untied output table), written by the
    reference on the spot."""
    spec = W.tiny(dtype, d_model=96, heads=6, kv_heads=2, hidden=160, vocab=131, layers=3, context=40, tied=tied)
    weights = W.make_weights(spec, seed=5)
    reference = oracle.CpuDecoder(spec, weights, kind="ref")
    model = B.DecoderModel(spec, weights, device=None)
    for with_head in (False, True):
        theirs, mine = str(tmp_path / "ref.onnx"), str(tmp_path / "mine.onnx")
        reference.save_onnx(theirs, with_head)
        model.save_onnx(mine, with_head)
        assert open(mine, "rb").read() == open(theirs, "rb").read(), (dtype, tied, with_head)


def test_export_argument_errors():
    spec = archive_cases()["micro_f32"]
    model = B.DecoderModel(spec, W.make_weights(spec, seed=77), device=None)
    l = B.lib()
    assert l.dl_onnx_save_decoder(b"/tmp/x.onnx", model.decoder.h, model.embedding.h, None) == 1
    assert b"both embedding and output" in l.dl_last_error()
    assert l.dl_onnx_save_decoder(b"/tmp/x.onnx", model.embedding.h, None, None) == 1
    assert b"not a TransformerDecoder" in l.dl_last_error()
    assert l.dl_onnx_save_decoder(b"/nonexistent-directory/x.onnx", model.decoder.h, None, None) == 1
    assert b"cannot write" in l.dl_last_error()


@pytest.mark.gpu
def test_export_from_device_resident_modules(tmp_path):
    """The same file when the weights live on the GPU (the exporter reads them back)."""
    spec = archive_cases()["micro_bf16"]
    model = B.DecoderModel(spec, W.make_weights(spec, seed=77))
    path = str(tmp_path / "device.onnx")
    model.save_onnx(path, True)
    assert open(path, "rb").read() == open(os.path.join(HERE, "golden", "micro_bf16_lm.onnx"), "rb").read()
