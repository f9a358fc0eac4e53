"""CPU tests: TRSH codec (golden bytes), bincode, TCP store semantics."""
import ctypes
import struct
import threading
import zlib

import pytest
import torch


def test_crc32_matches_zlib_polynomial():
    from torsh_b200.serialize import crc32
    for payload in (b"", b"123456789", bytes(range(256)) * 7):
        assert crc32(payload) == zlib.crc32(payload)
    assert crc32(b"123456789") == 0xCBF43926


def test_trsh_golden_layout():
    from torsh_b200.serialize import decode_trsh, encode_trsh
    t = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    b = encode_trsh(t, 0, {"k": "v"}, timestamp=300)
    assert b[:4] == b"TRSH" and struct.unpack("<I", b[4:8])[0] == 1
    ms, ds, crc = struct.unpack("<QQI", b[8:28])
    assert ds == 24 and len(b) == 28 + ms + ds
    meta = b[28:28 + ms]
    # shape [2,3] | Cpu | requires_grad false | "f32" | "0.1.3" | ts=300 (0xFB + u16) | {k:v} | "Binary" | 24 | false | None
    expect = bytes([2, 2, 3, 0, 0, 3]) + b"f32" + bytes([5]) + b"0.1.3" + bytes([251]) + struct.pack("<H", 300) + \
        bytes([1, 1]) + b"k" + bytes([1]) + b"v" + bytes([6]) + b"Binary" + bytes([24, 0, 0])
    assert meta == expect
    assert crc == zlib.crc32(b[28:])
    assert b[28 + ms:] == t.numpy().tobytes()
    t2, m = decode_trsh(b)
    assert torch.equal(t, t2) and m["custom_metadata"] == {"k": "v"} and m["format"] == "Binary"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.float16, torch.uint8])
@pytest.mark.parametrize("level", [0, 3])
def test_trsh_roundtrip(dtype, level, tmp_path):
    from torsh_b200.serialize import load_tensor, save_tensor
    t = (torch.randn(17, 5) * 10).to(dtype)
    save_tensor(t, tmp_path / "t.trsh", compression_level=level)
    assert torch.equal(load_tensor(tmp_path / "t.trsh"), t)
    if dtype == torch.float32:
        save_tensor(t, tmp_path / "t.json")
        assert torch.allclose(load_tensor(tmp_path / "t.json"), t)
        save_tensor(t, tmp_path / "t.npy")
        assert torch.equal(load_tensor(tmp_path / "t.npy"), t)


def test_trsh_rejects_corruption():
    from torsh_b200.core.error import TorshError
    from torsh_b200.serialize import decode_trsh, encode_trsh
    b = bytearray(encode_trsh(torch.ones(4)))
    b[-1] ^= 0xFF
    with pytest.raises(TorshError, match="checksum"):
        decode_trsh(bytes(b))
    with pytest.raises(TorshError, match="magic"):
        decode_trsh(b"NOPE" + bytes(40))


def test_bincode_python_matches_rules():
    from torsh_b200.serialize.bincode import Reader, Writer
    w = Writer()
    for v in (0, 250, 251, 65535, 65536, 2 ** 32 - 1, 2 ** 32, 2 ** 63):
        w.varu(v)
    for v in (0, -1, 1, -2 ** 40, 2 ** 40):
        w.vari(v)
    w.string("héllo")
    w.option(None, w.varu)
    w.option(7, w.varu)
    r = Reader(w.bytes())
    assert [r.varu() for _ in range(8)] == [0, 250, 251, 65535, 65536, 2 ** 32 - 1, 2 ** 32, 2 ** 63]
    assert [r.vari() for _ in range(5)] == [0, -1, 1, -2 ** 40, 2 ** 40]
    assert r.string() == "héllo" and r.option(r.varu) is None and r.option(r.varu) == 7 and r.remaining() == 0


def test_tcp_store_semantics():
    from torsh_b200.parallel.store import TCPStore
    server = TCPStore("127.0.0.1", 0, is_server=True)
    c1 = TCPStore("127.0.0.1", server.port)
    c2 = TCPStore("127.0.0.1", server.port)
    c1.set("a", b"hello")
    assert c2.get("a") == b"hello" and c2.get("missing") is None
    assert c2.contains("a") and not c2.contains("b") and c1.num_keys() == 1
    assert c1.add("ctr", 5) == 5 and c2.add("ctr", -2) == 3
    assert c1.compare_and_swap("a", b"nope", b"x") is False
    assert c1.compare_and_swap("a", b"hello", b"world") is True and c2.get("a") == b"world"
    assert c1.compare_and_swap("fresh", None, b"1") is True and c1.compare_and_swap("fresh", None, b"2") is False
    # wait blocks until another client sets the key
    t = threading.Timer(0.2, lambda: c2.set("late", b"1"))
    t.start()
    c1.wait(["late"], timeout=5.0)
    with pytest.raises(Exception):
        c1.wait(["never"], timeout=0.3)
    c1.set("ttl", b"x", ttl=0)
    assert c1.get("ttl") is None
    c1.delete("a")
    assert not c2.contains("a")
    for c in (c1, c2, server):
        c.close()
