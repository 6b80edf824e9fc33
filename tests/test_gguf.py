"""GGUF container reader (zq_gguf_*): header, metadata, tensor directory, errors - on the CPU; loading matrices, expert
slices, embedding rows and the LM-head arg-max - on the GPU, against the CPU oracle.

The file is written here the way the reference's own test writes its tiny GGUF (src/backend/cuda/expert.rs:928-952):
magic, version 3, counts, tensor directory with GGUF dimension order [columns, rows(, count)], payload aligned to 32."""
import struct

import numpy as np
import pytest

from tests import helpers as H


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors, metadata=(), version=3, alignment=None, magic=b"GGUF"):
    """tensors: list of (name, dims in GGUF order, type, payload bytes); metadata: list of (key, type id, packed value)."""
    head = bytearray(magic) + struct.pack("<I", version) + struct.pack("<QQ", len(tensors), len(metadata) + (1 if alignment else 0))
    for key, vt, packed in metadata:
        head += _s(key) + struct.pack("<I", vt) + packed
    if alignment:
        head += _s("general.alignment") + struct.pack("<I", 4) + struct.pack("<I", alignment)
    align = alignment or 32
    payload = bytearray()
    for name, dims, tt, data in tensors:
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<I", tt) + struct.pack("<Q", len(payload))
        payload += bytes(data)
        payload += b"\0" * (-len(payload) % align)
    head += b"\0" * (-len(head) % align)
    with open(path, "wb") as f:
        f.write(head + payload)


def _model(tmp_path, n_experts=3):
    rows, cols, inter = 64, 256, 96
    emb = H.random_weight(H.Q8_0, 50, cols, seed=1)
    head = H.random_weight(H.Q4_K, 200, cols, seed=2)
    gate = [H.random_weight(H.Q4_K, inter, cols, seed=10 + e) for e in range(n_experts)]
    down = [H.random_weight(H.Q5_0, cols, inter, seed=20 + e) for e in range(n_experts)]
    tensors = [
        ("token_embd.weight", [cols, 50], H.Q8_0, emb),
        ("output.weight", [cols, 200], H.Q4_K, head),
        ("blk.0.ffn_gate_exps.weight", [cols, inter, n_experts], H.Q4_K, np.concatenate(gate)),
        ("blk.0.ffn_down_exps.weight", [inter, cols, n_experts], H.Q5_0, np.concatenate(down)),
        ("blk.0.attn_norm.weight", [cols], 0, np.ones(cols, dtype=np.float32).tobytes()),
    ]
    meta = [("general.architecture", 8, _s("toy")), ("toy.block_count", 4, struct.pack("<I", 1)), ("toy.rope.freq_base", 6, struct.pack("<f", 10000.0)),
            ("tokenizer.ggml.tokens", 9, struct.pack("<IQ", 8, 3) + _s("a") + _s("b") + _s("c"))]
    path = tmp_path / "toy.gguf"
    write_gguf(path, tensors, meta)
    return path, dict(emb=emb, head=head, gate=gate, down=down, rows=rows, cols=cols, inter=inter)


def test_open_reads_directory_and_metadata(tmp_path):
    from zllm_b200.backend import GgufFile

    path, _ = _model(tmp_path)
    g = GgufFile(path)
    assert g.tensor_names() == ["token_embd.weight", "output.weight", "blk.0.ffn_gate_exps.weight", "blk.0.ffn_down_exps.weight", "blk.0.attn_norm.weight"]
    assert g.tensor_info("output.weight") == (H.Q4_K, [256, 200], 200 * 144)
    assert g.tensor_info("blk.0.ffn_gate_exps.weight") == (H.Q4_K, [256, 96, 3], 3 * 96 * 144)
    assert g.metadata_str("general.architecture") == "toy"
    assert g.metadata_u64("toy.block_count") == 1
    assert g.metadata_f64("toy.rope.freq_base") == 10000.0
    assert g.metadata_u64("tokenizer.ggml.tokens") == 3  # an array reports its length
    g.close()


def test_open_errors(tmp_path):
    from zllm_b200 import ffi
    from zllm_b200.backend import GgufFile

    good = [("w", [256, 2], H.Q4_K, bytes(288))]
    write_gguf(tmp_path / "magic.gguf", good, magic=b"GGML")
    write_gguf(tmp_path / "v2.gguf", good, version=2)
    write_gguf(tmp_path / "short.gguf", [("w", [256, 2], H.Q4_K, bytes(100))])      # payload shorter than the directory says
    write_gguf(tmp_path / "dup.gguf", good + good)
    write_gguf(tmp_path / "type.gguf", [("w", [256, 2], 99, bytes(288))])
    write_gguf(tmp_path / "blocks.gguf", [("w", [100, 2], H.Q4_K, bytes(288))])      # 200 elements are not whole blocks
    write_gguf(tmp_path / "align.gguf", good, alignment=24)
    for name in ("magic", "v2", "short", "dup", "type", "blocks", "align"):
        with pytest.raises(ffi.ZqFailure):
            GgufFile(tmp_path / f"{name}.gguf")
    with pytest.raises(ffi.ZqFailure):
        GgufFile(tmp_path / "missing.gguf")
    g = GgufFile(_model(tmp_path)[0])
    with pytest.raises(ffi.ZqFailure):
        g.tensor_info("no.such.tensor")
    with pytest.raises(ffi.ZqFailure):
        g.metadata_u64("general.architecture")  # a string


def test_split_files_are_opened_together(tmp_path):
    from zllm_b200 import ffi
    from zllm_b200.backend import GgufFile

    a = [("a.weight", [256, 2], H.Q4_K, bytes(288))]
    b = [("b.weight", [256, 4], H.Q4_K, bytes(576))]
    u16 = lambda v: struct.pack("<H", v)
    write_gguf(tmp_path / "m-00001-of-00002.gguf", a, [("split.count", 2, u16(2)), ("split.no", 2, u16(0)), ("split.tensors.count", 5, struct.pack("<i", 2))])
    write_gguf(tmp_path / "m-00002-of-00002.gguf", b, [("split.count", 2, u16(2)), ("split.no", 2, u16(1))])
    g = GgufFile(tmp_path / "m-00001-of-00002.gguf")
    assert g.tensor_names() == ["a.weight", "b.weight"]
    assert g.tensor_info("b.weight")[1] == [256, 4]
    write_gguf(tmp_path / "n-00001-of-00002.gguf", a, [("split.count", 2, u16(2))])
    with pytest.raises(ffi.ZqFailure):
        GgufFile(tmp_path / "n-00001-of-00002.gguf")  # the second shard is missing


@pytest.mark.gpu
def test_matrices_expert_slices_embedding_rows_and_lm_head(tmp_path):
    import torch

    from oracle import oracle as orc
    from tests.gpu_util import ctx, host
    from zllm_b200 import ffi
    from zllm_b200.backend import GgufFile, lm_head_argmax

    path, m = _model(tmp_path)
    g = GgufFile(path)
    c = ctx()
    cols, inter = m["cols"], m["inter"]
    head = g.load_matrix(c, "output.weight")
    assert (head.rows, head.cols, head.tensor_type) == (200, cols, H.Q4_K)
    want = orc.dequantize(H.Q4_K, m["head"], 200 * cols).reshape(200, cols)
    assert np.array_equal(host(c.dequantize(head)).view(np.uint32), want.view(np.uint32))
    for e in range(3):
        gate = g.load_matrix_slice(c, "blk.0.ffn_gate_exps.weight", e)
        down = g.load_matrix_slice(c, "blk.0.ffn_down_exps.weight", e)
        assert (gate.rows, gate.cols, down.rows, down.cols) == (inter, cols, cols, inter)
        assert np.array_equal(host(c.dequantize(gate)).view(np.uint32), orc.dequantize(H.Q4_K, m["gate"][e], inter * cols).reshape(inter, cols).view(np.uint32))
        assert np.array_equal(host(c.dequantize(down)).view(np.uint32), orc.dequantize(H.Q5_0, m["down"][e], inter * cols).reshape(cols, inter).view(np.uint32))
    with pytest.raises(ffi.ZqFailure):
        g.load_matrix_slice(c, "blk.0.ffn_gate_exps.weight", 3)
    with pytest.raises(ffi.ZqFailure):
        g.load_matrix(c, "blk.0.ffn_gate_exps.weight")  # three dimensions: not a matrix
    with pytest.raises(ffi.ZqFailure):
        g.load_matrix(c, "blk.0.attn_norm.weight")
    # embedding rows (GgufReader::embedding_rows, src/weight/container/gguf.rs:618-629): dequantised rows of the listed tokens
    emb = g.load_matrix(c, "token_embd.weight")
    ids = np.array([49, 0, 17], dtype=np.int32)
    rows = c.gather_rows(emb, torch.from_numpy(ids), dtype=torch.float32)
    c.sync()
    want = orc.dequantize(H.Q8_0, m["emb"], 50 * cols).reshape(50, cols)[ids]
    assert np.array_equal(rows.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # LM head + arg-max on the device against the oracle's logits
    x = np.random.default_rng(3).standard_normal((5, cols)).astype(np.float32)
    got = lm_head_argmax(c, head, torch.from_numpy(x).cuda())
    c.sync()
    logits = orc.linear(H.Q4_K, m["head"], 200, cols, x)
    assert list(got.cpu().numpy()) == list(np.argmax(logits, axis=1))


@pytest.mark.gpu
def test_argmax_rows_ties_and_nans():
    import torch

    from tests.gpu_util import ctx
    from zllm_b200 import ffi

    c = ctx()
    x = torch.zeros((4, 3000), device="cuda")
    x[0, 2999] = 1.0
    x[1, 7] = x[1, 1500] = 5.0           # a tie: the lower index wins
    x[2, :] = float("nan")               # nothing comparable: index 0
    x[3, 10] = float("nan")
    x[3, 2000] = -1.0
    x[3, :2000] = -2.0
    x[3, 2001:] = -2.0
    ids = torch.empty(4, dtype=torch.int32, device="cuda")
    import ctypes as C
    ffi.call("zq_argmax_rows", c.handle, C.c_void_p(x.data_ptr()), ffi.F32, 4, 3000, C.c_void_p(ids.data_ptr()))
    c.sync()
    assert list(ids.cpu().numpy()) == [2999, 7, 0, 2000]
