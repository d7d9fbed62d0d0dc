"""The source side of the loader on the CPU: manifest blocks, shuffle switches, epoch wrap, reset, node split and the
CPIO block cache (aeon src/manifest_file.cpp, src/block_manager.cpp:61-106, src/cache_system.cpp:69-146, src/cpio.cpp),
through the host-only stream handle of the C ABI."""
import ctypes as C
import json
import os
import struct

import pytest


def lib():
    from aeon_b200 import _lib as L
    return L, L.load()


class Stream:
    def __init__(self, cfg):
        self.L, self.l = lib()
        h = C.c_void_p()
        self.L.check(self.l.aeonb_stream_create(json.dumps(cfg).encode(), C.byref(h)))
        self.h = h
        rc, el, bc, st = C.c_int64(), C.c_int32(), C.c_int32(), C.c_int32()
        self.L.check(self.l.aeonb_stream_info(h, C.byref(rc), C.byref(el), C.byref(bc), C.byref(st), None, 0))
        self.records, self.elements, self.blocks = rc.value, el.value, bc.value

    def state(self):
        st = C.c_int32()
        d = C.create_string_buffer(512)
        self.L.check(self.l.aeonb_stream_info(self.h, None, None, None, C.byref(st), d, 512))
        return st.value, d.value.decode()

    def next(self):
        ptrs = (C.c_void_p * self.elements)()
        sizes = (C.c_size_t * self.elements)()
        self.L.check(self.l.aeonb_stream_next(self.h, ptrs, sizes))
        return tuple(C.string_at(ptrs[e], sizes[e]) for e in range(self.elements))

    def take(self, n):
        return [self.next() for _ in range(n)]

    def reset(self):
        self.L.check(self.l.aeonb_stream_reset(self.h))

    def close(self):
        if self.h:
            self.l.aeonb_stream_destroy(self.h)
            self.h = None


def write_manifest(tmp_path, n, files=False):
    lines = ["@FILE\tASCII_INT" if files else "@STRING\tASCII_INT"]
    for i in range(n):
        if files:
            (tmp_path / ("f%03d.bin" % i)).write_bytes(b"payload-%03d" % i + b"x" * (i % 3))
            lines.append("f%03d.bin\t%d" % (i, i))
        else:
            lines.append("rec%03d\t%d" % (i, i))
    path = tmp_path / "manifest.tsv"
    path.write_text("\n".join(lines) + "\n")
    return str(path)


def ids(records):
    return [struct.unpack("<i", r[1])[0] for r in records]


def test_plain_stream_keeps_manifest_order_and_wraps(tmp_path):
    s = Stream({"manifest_filename": write_manifest(tmp_path, 50), "batch_size": 4, "block_size": 10})
    assert (s.records, s.elements, s.blocks) == (50, 2, 5)
    got = s.take(120)
    assert ids(got) == [i % 50 for i in range(120)]
    assert got[7][0] == b"rec007"
    s.close()


def test_shuffle_enable_shuffles_inside_every_block_from_the_first_epoch(tmp_path):
    cfg = {"manifest_filename": write_manifest(tmp_path, 50), "batch_size": 4, "block_size": 10, "shuffle_enable": True,
           "random_seed": 7}
    a, b = Stream(cfg), Stream(cfg)
    e0 = ids(a.take(50))
    assert e0 != list(range(50))                                  # already the first epoch is shuffled
    for k in range(5):                                            # ... inside each block, blocks in manifest order
        assert sorted(e0[10 * k:10 * k + 10]) == list(range(10 * k, 10 * k + 10))
    e1 = ids(a.take(50))
    assert sorted(e1) == list(range(50)) and e1 != e0             # the generator moves on from epoch to epoch
    assert ids(b.take(100)) == e0 + e1                            # same seed, same stream
    # reset goes back to block 0 and keeps the generator's state: two loaders doing the same calls see the same records
    a.reset(), b.reset()
    r = ids(a.take(30))
    assert ids(b.take(30)) == r and sorted(r[:10]) == list(range(10))
    a.close(), b.close()


def test_shuffle_manifest_shuffles_records_once_and_block_order_on_wrap(tmp_path):
    cfg = {"manifest_filename": write_manifest(tmp_path, 40), "batch_size": 4, "block_size": 10, "shuffle_manifest": True,
           "random_seed": 3}
    a = Stream(cfg)
    e0, e1 = ids(a.take(40)), ids(a.take(40))
    assert sorted(e0) == list(range(40)) and e0 != list(range(40))
    blocks0 = [e0[10 * k:10 * k + 10] for k in range(4)]
    blocks1 = [e1[10 * k:10 * k + 10] for k in range(4)]
    assert sorted(map(tuple, blocks0)) == sorted(map(tuple, blocks1))   # the blocks stay, only their order changes
    b = Stream(cfg)
    assert ids(b.take(80)) == e0 + e1
    a.close(), b.close()


def test_node_split_matches_the_reference_test(tmp_path):
    """aeon test/test_manifest_tsv.cpp:113-205: interleaved batch slices, evenly divided tail."""
    from aeon_b200.sharding import shard_indices
    assert shard_indices(10, 3, 0, 2) == [0, 1, 2, 6, 7] and shard_indices(10, 3, 1, 2) == [3, 4, 5, 8, 9]
    path = write_manifest(tmp_path, 10)
    got = []
    for node in range(2):
        s = Stream({"manifest_filename": path, "batch_size": 3, "node_id": node, "node_count": 2})
        assert s.records == 5
        got.append(ids(s.take(5)))
        s.close()
    assert got == [[0, 1, 2, 6, 7], [3, 4, 5, 8, 9]]


def parse_cpio(path):
    """Independent reader of aeon's block file layout: old binary cpio members around a 64-byte 'MACR' header."""
    data = open(path, "rb").read()
    at, members = 0, []
    while at < len(data):
        f = struct.unpack_from("<13H", data, at)
        assert f[0] == 0o70707 and f[3] == 0o100644
        namesize, size = f[10], (f[11] << 16) | f[12]
        at += 26
        name = data[at:at + namesize - 1].decode()
        at += namesize + (namesize & 1)
        members.append((name, data[at:at + size]))
        at += size + (size & 1)
    return members


def test_cpio_cache_is_written_once_then_read_instead_of_the_files(tmp_path):
    cache = tmp_path / "cache"
    cache.mkdir()
    cfg = {"manifest_filename": write_manifest(tmp_path, 25, files=True), "manifest_root": str(tmp_path), "batch_size": 4,
           "block_size": 10, "cache_directory": str(cache)}
    a = Stream(cfg)
    state, directory = a.state()
    assert state == 2 and os.path.basename(directory).startswith("aeon_cache_") and os.path.isfile(directory + "/caching_in_progress")
    busy = Stream(cfg)                      # a second loader while the first one is still writing
    assert busy.state()[0] == 1
    first = a.take(25)
    assert ids(first) == list(range(25)) and first[3][0] == b"payload-003"
    assert a.state()[0] == 3 and os.path.isfile(directory + "/cache_complete") and not os.path.exists(directory + "/caching_in_progress")
    assert sorted(f for f in os.listdir(directory) if f.endswith(".cpio")) == ["block_0.cpio", "block_1.cpio", "block_2.cpio"]
    assert ids(busy.take(25)) == list(range(25))   # the blocked loader read the files itself
    busy.close()
    # the block files follow aeon's layout
    m = parse_cpio(directory + "/block_1.cpio")
    assert [n for n, _ in m][:3] == ["cpiohdr", "rec_0000000.00", "rec_0000000.01"] and [n for n, _ in m][-2:] == ["cpiotlr", "TRAILER!!!"]
    head = m[0][1]
    assert head[:4] == b"MACR" and struct.unpack_from("<II", head, 4) == (1, 1) and struct.unpack_from("<I", head, 20)[0] == 9
    assert m[1][1] == b"payload-009" and struct.unpack("<i", m[2][1])[0] == 9      # block 1 starts at record 9 (25 records in 3 blocks)
    # from now on nothing touches the source files: remove them and read two more epochs, also from a new loader
    for i in range(25):
        os.remove(tmp_path / ("f%03d.bin" % i))
    assert ids(a.take(50)) == list(range(25)) * 2
    b = Stream(cfg)
    assert b.state()[0] == 3 and b.take(25) == first
    a.close(), b.close()
    # a damaged block file is reported, not silently skipped
    open(directory + "/block_0.cpio", "wb").write(b"junk")
    c = Stream(cfg)
    from aeon_b200._lib import AeonError
    with pytest.raises(AeonError, match="CPIO|cache"):
        c.take(1)
    c.close()


def test_shuffled_cache_reads_permute_blocks_and_records(tmp_path):
    cache = tmp_path / "cache"
    cache.mkdir()
    cfg = {"manifest_filename": write_manifest(tmp_path, 30), "batch_size": 4, "block_size": 10, "cache_directory": str(cache),
           "shuffle_enable": True, "random_seed": 11}
    a = Stream(cfg)
    e0 = ids(a.take(30))            # written to the cache unshuffled, handed out shuffled inside the blocks
    assert [sorted(e0[10 * k:10 * k + 10]) for k in range(3)] == [list(range(10 * k, 10 * k + 10)) for k in range(3)]
    d = a.state()[1]
    assert [struct.unpack("<i", v)[0] for n, v in parse_cpio(d + "/block_0.cpio") if n.endswith(("1", "3", "5", "7", "9")) and n.startswith("rec")] == list(range(10))
    e1 = ids(a.take(30))            # now from the cache: block order and block contents shuffled
    assert sorted(e1) == list(range(30))
    assert all(len({v // 10 for v in e1[10 * k:10 * k + 10]}) == 1 for k in range(3))
    a.close()


def test_large_blocks_are_read_by_several_threads_and_one_block_ahead(tmp_path):
    """A block of a few hundred file records goes through the parallel readers (small blocks are read by the calling thread):
    same records, same order; the cache written from it reads back the same; a file that disappears is reported by the call
    that needs its block, with the reference's message, and the stream does not hang."""
    n = 600
    cache = tmp_path / "cache"
    cache.mkdir()
    cfg = {"manifest_filename": write_manifest(tmp_path, n, files=True), "manifest_root": str(tmp_path), "batch_size": 8,
           "block_size": 250}
    a = Stream(cfg)
    first = a.take(2 * n)
    assert ids(first) == list(range(n)) * 2 and first[417][0] == b"payload-417" + b"x" * (417 % 3)
    a.close()
    b = Stream(dict(cfg, cache_directory=str(cache)))
    assert b.take(n) == first[:n]            # written to the cache on the way
    assert b.state()[0] == 3
    assert b.take(2 * n) == first            # read back from the CPIO blocks by the parallel reader
    b.close()
    os.remove(tmp_path / "f300.bin")          # second block of a stream without cache
    c = Stream(cfg)
    assert ids(c.take(200)) == list(range(200))
    from aeon_b200._lib import AeonError
    with pytest.raises(AeonError, match="error opening file"):
        c.take(200)
    c.close()
