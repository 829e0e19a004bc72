"""MoE block of the engine's checkpoint file (host code of the library; no GPU).

The stock part of the file is built here the way the engine's writer lays it out
(core/src/training.cpp:283-392): 56-byte header "AXIOM_V1" + six u64, fp32 weights, bias,
embeddings, then the transformer block (u64 tag 0x5458464D, u64 dim, u64 ffn, four dim x dim
and three dim x ffn fp32 matrices).  The tests mirror the engine's own corrupt-file tests
(core/test/test_inference.cpp:369-448): truncated files, wrong tags and non-finite values
are refused, and a refused save leaves the original file untouched.
"""
import importlib
import os
import struct

import numpy as np
import pytest

XFORM_TAG = 0x5458464D
MOE_TAG = 0x4D4F4558


@pytest.fixture(scope="module")
def ckpt(axm):
    return importlib.import_module("project_axiom_ai_llm_b200.checkpoint")


def stock_file(path, rng, with_xform=True, in_total=6, out_total=4, vocab=5, dim=4, ffn=8):
    """A small checkpoint as the engine writes it; returns its bytes."""
    header = b"AXIOM_V1" + struct.pack("<6Q", in_total, out_total, in_total * out_total, out_total, vocab, out_total)
    body = rng.standard_normal(in_total * out_total + out_total + vocab * out_total).astype(np.float32).tobytes()
    blob = header + body
    if with_xform:
        blob += struct.pack("<3Q", XFORM_TAG, dim, ffn)
        blob += rng.standard_normal(4 * dim * dim + 3 * dim * ffn).astype(np.float32).tobytes()
    with open(path, "wb") as f:
        f.write(blob)
    return blob


def moe_weights(rng, D=8, F=16, E=4, S=0, bias=False):
    w = {"router_w": rng.standard_normal((D, E)).astype(np.float32),
         "w_gate": rng.standard_normal((E, D, F)).astype(np.float32),
         "w_up": rng.standard_normal((E, D, F)).astype(np.float32),
         "w_down": rng.standard_normal((E, F, D)).astype(np.float32)}
    if bias:
        w["router_bias"] = rng.standard_normal(E).astype(np.float32)
    if S:
        w["shared_gate"] = rng.standard_normal((S, D, F)).astype(np.float32)
        w["shared_up"] = rng.standard_normal((S, D, F)).astype(np.float32)
        w["shared_down"] = rng.standard_normal((S, F, D)).astype(np.float32)
    return w


@pytest.mark.parametrize("S,bias", [(0, False), (2, True)])
def test_round_trip_keeps_the_stock_payload(ckpt, tmp_path, S, bias):
    rng = np.random.default_rng(1)
    path = str(tmp_path / "weights.axiom")
    stock = stock_file(path, rng)
    w = moe_weights(rng, S=S, bias=bias)
    ckpt.save_moe_block(path, w, top_k=2)
    blob = open(path, "rb").read()
    assert blob[:len(stock)] == stock, "the engine's own payload must survive byte for byte"
    assert struct.unpack("<Q", blob[len(stock):len(stock) + 8])[0] == MOE_TAG
    assert not os.path.exists(path + ".tmp")
    info, got = ckpt.load_moe_block(path)
    assert info == {"d_model": 8, "d_ff": 16, "num_experts": 4, "top_k": 2, "num_shared": S, "router_bias": bias}
    assert set(got) == set(w)
    for n in w:
        assert np.array_equal(got[n], w[n]), n


def test_second_save_replaces_the_block(ckpt, tmp_path):
    rng = np.random.default_rng(2)
    path = str(tmp_path / "weights.axiom")
    stock = stock_file(path, rng)
    ckpt.save_moe_block(path, moe_weights(rng), top_k=2)
    size_one = os.path.getsize(path)
    w2 = moe_weights(rng, D=8, F=16, E=4)
    ckpt.save_moe_block(path, w2, top_k=1)
    assert os.path.getsize(path) == size_one
    info, got = ckpt.load_moe_block(path)
    assert info["top_k"] == 1 and np.array_equal(got["w_down"], w2["w_down"])
    assert open(path, "rb").read()[:len(stock)] == stock


def test_block_layout_on_disk(ckpt, tmp_path):
    rng = np.random.default_rng(3)
    path = str(tmp_path / "weights.axiom")
    stock = stock_file(path, rng)
    w = moe_weights(rng, D=4, F=8, E=2, bias=True)
    ckpt.save_moe_block(path, w, top_k=2)
    blob = open(path, "rb").read()[len(stock):]
    head = struct.unpack("<9Q", blob[:72])
    payload = b"".join(w[n].tobytes() for n in ("router_w", "router_bias", "w_gate", "w_up", "w_down"))
    assert head == (MOE_TAG, 1, 4, 8, 2, 2, 0, 1, len(payload))
    assert blob[72:72 + len(payload)] == payload
    checksum = int(np.frombuffer(payload, dtype="<u4").astype(np.uint64).sum())
    assert struct.unpack("<Q", blob[72 + len(payload):])[0] == checksum
    assert len(blob) == 72 + len(payload) + 8


def test_refuses_non_finite_and_leaves_the_file_alone(ckpt, axm, tmp_path):
    rng = np.random.default_rng(4)
    path = str(tmp_path / "weights.axiom")
    stock = stock_file(path, rng)
    w = moe_weights(rng)
    w["w_up"][1, 2, 3] = np.nan
    with pytest.raises(axm.AxmError, match="w_up contains NaN or Inf"):
        ckpt.save_moe_block(path, w, top_k=2)
    assert open(path, "rb").read() == stock and not os.path.exists(path + ".tmp")


def test_needs_a_transformer_block(ckpt, axm, tmp_path):
    rng = np.random.default_rng(5)
    path = str(tmp_path / "weights.axiom")
    stock = stock_file(path, rng, with_xform=False)
    with pytest.raises(axm.AxmError, match="no transformer block"):
        ckpt.save_moe_block(path, moe_weights(rng), top_k=2)
    assert open(path, "rb").read() == stock
    with pytest.raises(axm.AxmError):
        ckpt.probe_moe_block(path)


def test_rejects_foreign_and_damaged_files(ckpt, axm, tmp_path):
    rng = np.random.default_rng(6)
    path = str(tmp_path / "weights.axiom")
    with pytest.raises(axm.AxmError, match="cannot open"):
        ckpt.probe_moe_block(path)
    open(path, "wb").write(b"NOTAXIOM" + bytes(100))
    with pytest.raises(axm.AxmError, match="not an AXIOM_V1"):
        ckpt.save_moe_block(path, moe_weights(rng), top_k=2)
    stock = stock_file(path, rng)
    with pytest.raises(axm.AxmError, match="holds no MoE block"):
        ckpt.load_moe_block(path)
    ckpt.save_moe_block(path, moe_weights(rng), top_k=2)
    good = open(path, "rb").read()
    # truncated in the payload
    open(path, "wb").write(good[:-40])
    with pytest.raises(axm.AxmError, match="incomplete"):
        ckpt.load_moe_block(path)
    # one flipped payload bit: sizes are fine, the checksum is not
    bad = bytearray(good)
    bad[len(stock) + 72 + 5] ^= 0x10
    open(path, "wb").write(bytes(bad))
    with pytest.raises(axm.AxmError, match="checksum"):
        ckpt.load_moe_block(path)
    # unknown tag where the block should start
    bad = bytearray(good)
    bad[len(stock)] ^= 0xFF
    open(path, "wb").write(bytes(bad))
    with pytest.raises(axm.AxmError, match="unknown tag"):
        ckpt.probe_moe_block(path)
    # a truncated transformer block
    open(path, "wb").write(stock[:-12])
    with pytest.raises(axm.AxmError, match="transformer block"):
        ckpt.save_moe_block(path, moe_weights(rng), top_k=2)


def test_load_checks_the_layer_shape(ckpt, axm, tmp_path):
    import ctypes
    rng = np.random.default_rng(7)
    path = str(tmp_path / "weights.axiom")
    stock_file(path, rng)
    w = moe_weights(rng)
    ckpt.save_moe_block(path, w, top_k=2)
    desc = axm.make_desc(0, 8, 16, 8, 2)  # the file has 4 experts
    table = axm.MoeCheckpoint()
    rc = axm.load().axm_moe_checkpoint_load(os.fsencode(path), ctypes.byref(desc), ctypes.byref(table))
    assert rc == axm.AXM_ERR_ARGUMENT and b"4 experts" in axm.load().axm_last_error()
    desc = axm.make_desc(0, 8, 16, 4, 2)  # right shape, missing buffers
    rc = axm.load().axm_moe_checkpoint_load(os.fsencode(path), ctypes.byref(desc), ctypes.byref(table))
    assert rc == axm.AXM_ERR_ARGUMENT and b"router_w is null" in axm.load().axm_last_error()


def test_shape_mismatch_is_a_python_error(ckpt, tmp_path):
    rng = np.random.default_rng(8)
    path = str(tmp_path / "weights.axiom")
    stock_file(path, rng)
    w = moe_weights(rng)
    w["w_down"] = w["w_down"][:, :, :-1]
    with pytest.raises(ValueError, match="w_down"):
        ckpt.save_moe_block(path, w, top_k=2)
