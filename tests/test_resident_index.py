"""The resident weight file's index reader (host code behind the C ABI) against the reference reader's own test
cases: hand-assembled fixtures of the documented header / entry / name layout
(crates/model-io/tests/resident_index.rs:15-300)."""
import struct

import pytest

HEADER_BYTES, ENTRY_BYTES, TRAILER_BYTES = 24, 72, 16
MAGIC, VERSION = b"GTURBIDX", 1


def build_index_bytes(name, trailer=None):
    # crates/model-io/tests/resident_index.rs:21-72: one BF16 64x64 entry; legacy layout unless a trailer is asked for
    nb = name if isinstance(name, bytes) else name.encode()
    name_offset = HEADER_BYTES + ENTRY_BYTES
    string_end = name_offset + len(nb)
    index_size = string_end + 7 + TRAILER_BYTES if trailer is not None else string_end
    buf = bytearray(struct.pack("<QQQ", index_size, 4096, 1))
    buf += struct.pack("<IHBBQQ4IQQQQ", name_offset, len(nb), 1, 0, index_size, 4096, 64, 64, 1, 1, 0, 0, 0, 0)
    buf += nb
    if trailer is not None:
        buf += bytes(7) + MAGIC + struct.pack("<II", trailer, 0)
    assert len(buf) == index_size
    buf += bytes(4096)
    return buf


def set_u64(buf, field_offset, value):
    buf[HEADER_BYTES + field_offset:HEADER_BYTES + field_offset + 8] = struct.pack("<Q", value)


@pytest.fixture
def opener(tmp_path):
    from turbospark_b200 import resident
    counter = [0]

    def open_bytes(data):
        counter[0] += 1
        p = tmp_path / ("w%d.bin" % counter[0])
        p.write_bytes(bytes(data))
        return resident.ResidentIndex(p)
    return open_bytes, resident


def test_legacy_index_without_a_trailer_loads_and_one_entry_parses(opener):
    open_bytes, _ = opener
    idx = open_bytes(build_index_bytes("blk.0.attn.q_proj"))
    assert len(idx) == 1 and idx.names() == ["blk.0.attn.q_proj"]
    e = idx.find("blk.0.attn.q_proj")
    assert e.dtype == 1 and tuple(e.shape) == (64, 64, 1, 1) and e.size_bytes == 4096
    assert idx.index_size == HEADER_BYTES + ENTRY_BYTES + len("blk.0.attn.q_proj") and idx.data_size == 4096
    assert e.file_offset == idx.index_size


def test_trailer_naming_the_supported_format_loads_and_an_unknown_one_is_refused_by_name(opener):
    open_bytes, resident = opener
    assert len(open_bytes(build_index_bytes("w", trailer=VERSION))) == 1
    with pytest.raises(resident.ResidentError) as ei:
        open_bytes(build_index_bytes("w", trailer=VERSION + 1))
    assert ei.value.code == 3 and "index format 2 is not supported" in ei.value.message


def test_magic_inside_the_string_table_is_not_a_trailer(opener):
    open_bytes, _ = opener
    name = b"x." + MAGIC + struct.pack("<II", VERSION + 1, 0)
    idx = open_bytes(build_index_bytes(name))
    assert len(idx) == 1


def test_corrupt_indexes_are_refused(opener):
    open_bytes, resident = opener

    def refused(data, needle="index corrupt"):
        with pytest.raises(resident.ResidentError) as ei:
            open_bytes(data)
        assert ei.value.code == 1 and needle in ei.value.message, ei.value.message

    refused(bytes(4))                                             # short header
    b = build_index_bytes("x")
    b[HEADER_BYTES + 4:HEADER_BYTES + 6] = struct.pack("<H", 9999)
    refused(b, "name range")                                      # name past the index region
    b = build_index_bytes("x")
    b[16:24] = struct.pack("<Q", 2 ** 64 - 2)
    refused(b, "overflows")                                       # entry count that overflows the table size
    b = build_index_bytes("x")
    b[0:8] = struct.pack("<Q", 1 << 40)
    refused(b)                                                    # index size past the end of the file
    b = build_index_bytes("x")
    set_u64(b, 16, 4096 * 10)
    refused(b, "payload")                                         # payload past the resident region
    b = build_index_bytes("x")
    set_u64(b, 40, 1 << 20)
    set_u64(b, 48, 64)
    refused(b, "scale")                                           # scale plane past the resident region
    b = build_index_bytes("x")
    set_u64(b, 8, 0)
    refused(b, "payload")                                         # payload offset inside the index region


def test_affine_entries_must_carry_planes_of_the_declared_shape(opener):
    open_bytes, resident = opener
    b = build_index_bytes("x")
    b[HEADER_BYTES + 6] = 4
    set_u64(b, 16, 2048), set_u64(b, 40, 96 + 2048), set_u64(b, 48, 2), set_u64(b, 56, 96 + 2050), set_u64(b, 64, 2)
    with pytest.raises(resident.ResidentError) as ei:
        open_bytes(b)
    assert "affine planes" in ei.value.message
    b = build_index_bytes("x")
    b[HEADER_BYTES + 6] = 4
    b[HEADER_BYTES + 24:HEADER_BYTES + 28] = struct.pack("<I", 999)
    with pytest.raises(resident.ResidentError):
        open_bytes(b)
    b = build_index_bytes("x")
    b[HEADER_BYTES + 6] = 4
    set_u64(b, 16, 2048), set_u64(b, 40, 97), set_u64(b, 48, 128), set_u64(b, 56, 224), set_u64(b, 64, 128)
    with pytest.raises(resident.ResidentError):
        open_bytes(b)


def test_the_writer_lays_files_out_as_the_reference_writer_does(opener):
    # crates/repack/src/resident_writer.rs:375-470: page-rounded index with the trailer in its last 16 bytes,
    # entries 4-byte aligned, payload offsets absolute
    open_bytes, resident = opener
    data = resident.build_resident_file([("a.weight", 7, (1, 256, 1, 1), bytes(range(144))),
                                         ("n", 1, (3, 1, 1, 1), b"\x01\x02\x03\x04\x05\x06"),
                                         ("b.weight", 8, (1, 256, 1, 1), bytes(210))])
    assert data[resident.PAGE_BYTES - 16:resident.PAGE_BYTES - 8] == MAGIC
    idx = open_bytes(data)
    assert idx.index_size == resident.PAGE_BYTES and idx.names() == ["a.weight", "n", "b.weight"]
    a, n, b = idx.find("a.weight"), idx.find("n"), idx.find("b.weight")
    assert a.file_offset == resident.PAGE_BYTES and n.file_offset == a.file_offset + 144
    assert b.file_offset == n.file_offset + 8 and b.file_offset % 4 == 0     # 6 bytes of norm, padded to 4
    assert data[a.file_offset:a.file_offset + 144] == bytes(range(144))
    assert idx.data_size == 144 + 8 + 210
    with pytest.raises(resident.ResidentError):
        idx.find("missing")
    from turbospark_b200 import lib
    assert [lib().tsb_resident_qtype_of(t) for t in (7, 8, 14, 13, 6, 1)] == [0, 1, 2, 3, 4, -1]
