"""Weight archives (".ct"): dl_state_load / dl_state_save against files written by the UNMODIFIED reference library
(tests/golden/*.ct, made by tests/golden/make_golden.py) — layout of src/io/checkpoint.cpp:52-114 of the reference."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))

import ctorch_b200 as B
import oracle
from cases import archive_cases
from ctorch_b200 import workloads as W

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def expected_entries(spec):
    """(name, array) the reference's example model holds for these seeded weights: the parameters in registration order,
    each attention followed by its two RoPE buffers (tokens first, then the decoder's state under "decoder.")."""
    named = dict(zip([n for n, _ in W.tensor_shapes(spec)], W.make_weights(spec, seed=77)))
    return named


@pytest.mark.parametrize("name", list(archive_cases()))
def test_reads_reference_archive(name):
    spec = archive_cases()[name]
    state = B.load_archive(os.path.join(GOLDEN, name + ".ct"))
    want = expected_entries(spec)
    assert set(want) <= set(state)
    extra = sorted(set(state) - set(want))
    assert extra and all(n.endswith("rotary.cosine") or n.endswith("rotary.sine") for n in extra)
    code = B.BF16 if spec["dtype"] == "bf16" else B.F32
    for key, array in want.items():
        t = state[key]
        assert t.dtype == code and t.shape == array.shape, key
        assert np.array_equal(t.numpy(), array), key
    cos, sin = oracle.rope_tables(spec["d_model"] // spec["heads"], spec["context"], spec["rope_base"])
    assert np.array_equal(state["decoder.layer0.attention.rotary.cosine"].numpy(), cos)
    assert np.array_equal(state["decoder.layer1.attention.rotary.sine"].numpy(), sin)


@pytest.mark.parametrize("name", list(archive_cases()))
def test_written_archive_is_byte_identical_to_the_reference_file(name, tmp_path):
    source = os.path.join(GOLDEN, name + ".ct")
    state = B.load_archive(source)
    target = tmp_path / "copy.ct"
    B.save_archive(target, state)
    assert target.read_bytes() == open(source, "rb").read()
    assert not (tmp_path / "copy.ct.partial").exists()


def test_rejects_foreign_and_truncated_files(tmp_path):
    bad = tmp_path / "bad.ct"
    bad.write_bytes(b"NOTCTORCH" + bytes(64))
    with pytest.raises(B.B200Error, match="unsupported Ctorch checkpoint format"):
        B.load_archive(bad)
    whole = open(os.path.join(GOLDEN, "micro_f32.ct"), "rb").read()
    cut = tmp_path / "cut.ct"
    cut.write_bytes(whole[: len(whole) // 2])
    with pytest.raises(B.B200Error):
        B.load_archive(cut)
    huge = tmp_path / "huge.ct"
    huge.write_bytes(whole[:8] + (2 ** 60).to_bytes(8, "little") + whole[16:64])
    with pytest.raises(B.B200Error, match="corrupt"):
        B.load_archive(huge)


@pytest.mark.skipif(not oracle.have_ref(), reason="reference library not built on this machine")
def test_reference_reads_what_this_library_writes(tmp_path):
    rng = np.random.default_rng(3)
    named = {"a.weight": B.Tensor.from_numpy(rng.standard_normal((3, 5), dtype=np.float32)),
             "b": B.Tensor.from_numpy(W.bf16_bits(rng.standard_normal((4,), dtype=np.float32)), dtype=B.BF16),
             "ids": B.Tensor.from_numpy(np.arange(6, dtype=np.int64).reshape(2, 3))}
    path = tmp_path / "mine.ct"
    B.save_archive(path, named)
    entries = oracle.reference_archive(str(path))
    assert [e[0] for e in entries] == list(named)
    for (name, shape, dtype, data), tensor in zip(entries, named.values()):
        assert shape == tensor.shape and dtype == tensor.dtype
        assert data == tensor.numpy().tobytes()


@pytest.mark.gpu
def test_decoder_loaded_from_archive_matches_oracle():
    spec = archive_cases()["micro_bf16"]
    weights = W.make_weights(spec, seed=77)
    model = B.DecoderModel(spec, [np.zeros_like(w) for w in weights])       # wrong weights first
    state = B.load_archive(os.path.join(GOLDEN, "micro_bf16.ct"))
    model.load_archive_state(state)
    prompt = W.make_prompts(spec, seed=5)
    cpu = oracle.CpuDecoder(spec, weights)
    want = cpu.decode_ids(prompt)
    got = model.decode_ids(prompt)
    assert np.abs(got - want).max() / np.abs(want).max() < 2e-2
