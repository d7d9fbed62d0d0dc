"""CPU oracle for baseline JPEG decoding as ``cv::imdecode`` performs it (TEST INFRASTRUCTURE ONLY).

aeon decodes every image and video frame with ``cv::imdecode`` (src/etl_image.cpp:90,
src/cap_mjpeg_decoder.cpp:140).  OpenCV hands JPEG data to libjpeg / libjpeg-turbo (the
binary in this environment bundles libjpeg-turbo 3.1.2), neither of which is part of
the aeon tree.  This module restates the published algorithms that library applies with
its default settings and is pinned bit-for-bit against ``cv2.imdecode``:

* ITU-T T.81 baseline sequential entropy decoding (Huffman, restart intervals);
* dequantisation and the 8x8 "slow integer" inverse DCT: the Loeffler-Ligtenberg-Moschytz
  factorisation with 13-bit constants, 2 extra bits kept after the column pass, results
  level-shifted by 128 and clamped to 0..255;
* "fancy" (triangle-filter) chroma upsampling for 2x1 and 2x2 subsampled components;
* JFIF YCbCr -> RGB with 16-bit fixed-point constants.

The entropy decoder is written as plain Python loops and is meant for small images only.
Nothing in the shipped package imports this file.
"""
import numpy as np

ZIGZAG = np.array([
    0, 1, 8, 16, 9, 2, 3, 10, 17, 24, 32, 25, 18, 11, 4, 5, 12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13, 6, 7, 14, 21, 28,
    35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47,
    55, 62, 63])

# ITU-T T.81 Annex K.3 typical Huffman tables; MJPEG frames may omit their DHT segments and rely on these.
STD_DC_LUMA = ([0, 1, 5, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 0], list(range(12)))
STD_DC_CHROMA = ([0, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0], list(range(12)))
STD_AC_LUMA = ([0, 2, 1, 3, 3, 2, 4, 3, 5, 5, 4, 4, 0, 0, 1, 0x7d], [
    0x01, 0x02, 0x03, 0x00, 0x04, 0x11, 0x05, 0x12, 0x21, 0x31, 0x41, 0x06, 0x13, 0x51, 0x61, 0x07, 0x22, 0x71, 0x14, 0x32,
    0x81, 0x91, 0xa1, 0x08, 0x23, 0x42, 0xb1, 0xc1, 0x15, 0x52, 0xd1, 0xf0, 0x24, 0x33, 0x62, 0x72, 0x82, 0x09, 0x0a, 0x16,
    0x17, 0x18, 0x19, 0x1a, 0x25, 0x26, 0x27, 0x28, 0x29, 0x2a, 0x34, 0x35, 0x36, 0x37, 0x38, 0x39, 0x3a, 0x43, 0x44, 0x45,
    0x46, 0x47, 0x48, 0x49, 0x4a, 0x53, 0x54, 0x55, 0x56, 0x57, 0x58, 0x59, 0x5a, 0x63, 0x64, 0x65, 0x66, 0x67, 0x68, 0x69,
    0x6a, 0x73, 0x74, 0x75, 0x76, 0x77, 0x78, 0x79, 0x7a, 0x83, 0x84, 0x85, 0x86, 0x87, 0x88, 0x89, 0x8a, 0x92, 0x93, 0x94,
    0x95, 0x96, 0x97, 0x98, 0x99, 0x9a, 0xa2, 0xa3, 0xa4, 0xa5, 0xa6, 0xa7, 0xa8, 0xa9, 0xaa, 0xb2, 0xb3, 0xb4, 0xb5, 0xb6,
    0xb7, 0xb8, 0xb9, 0xba, 0xc2, 0xc3, 0xc4, 0xc5, 0xc6, 0xc7, 0xc8, 0xc9, 0xca, 0xd2, 0xd3, 0xd4, 0xd5, 0xd6, 0xd7, 0xd8,
    0xd9, 0xda, 0xe1, 0xe2, 0xe3, 0xe4, 0xe5, 0xe6, 0xe7, 0xe8, 0xe9, 0xea, 0xf1, 0xf2, 0xf3, 0xf4, 0xf5, 0xf6, 0xf7, 0xf8,
    0xf9, 0xfa])
STD_AC_CHROMA = ([0, 2, 1, 2, 4, 4, 3, 4, 7, 5, 4, 4, 0, 1, 2, 0x77], [
    0x00, 0x01, 0x02, 0x03, 0x11, 0x04, 0x05, 0x21, 0x31, 0x06, 0x12, 0x41, 0x51, 0x07, 0x61, 0x71, 0x13, 0x22, 0x32, 0x81,
    0x08, 0x14, 0x42, 0x91, 0xa1, 0xb1, 0xc1, 0x09, 0x23, 0x33, 0x52, 0xf0, 0x15, 0x62, 0x72, 0xd1, 0x0a, 0x16, 0x24, 0x34,
    0xe1, 0x25, 0xf1, 0x17, 0x18, 0x19, 0x1a, 0x26, 0x27, 0x28, 0x29, 0x2a, 0x35, 0x36, 0x37, 0x38, 0x39, 0x3a, 0x43, 0x44,
    0x45, 0x46, 0x47, 0x48, 0x49, 0x4a, 0x53, 0x54, 0x55, 0x56, 0x57, 0x58, 0x59, 0x5a, 0x63, 0x64, 0x65, 0x66, 0x67, 0x68,
    0x69, 0x6a, 0x73, 0x74, 0x75, 0x76, 0x77, 0x78, 0x79, 0x7a, 0x82, 0x83, 0x84, 0x85, 0x86, 0x87, 0x88, 0x89, 0x8a, 0x92,
    0x93, 0x94, 0x95, 0x96, 0x97, 0x98, 0x99, 0x9a, 0xa2, 0xa3, 0xa4, 0xa5, 0xa6, 0xa7, 0xa8, 0xa9, 0xaa, 0xb2, 0xb3, 0xb4,
    0xb5, 0xb6, 0xb7, 0xb8, 0xb9, 0xba, 0xc2, 0xc3, 0xc4, 0xc5, 0xc6, 0xc7, 0xc8, 0xc9, 0xca, 0xd2, 0xd3, 0xd4, 0xd5, 0xd6,
    0xd7, 0xd8, 0xd9, 0xda, 0xe2, 0xe3, 0xe4, 0xe5, 0xe6, 0xe7, 0xe8, 0xe9, 0xea, 0xf2, 0xf3, 0xf4, 0xf5, 0xf6, 0xf7, 0xf8,
    0xf9, 0xfa])


class JpegError(RuntimeError):
    pass


class _Huff:
    def __init__(self, bits, vals):
        self.lookup = {}
        code = 0
        k = 0
        for length in range(1, 17):
            for _ in range(bits[length - 1]):
                self.lookup[(length, code)] = vals[k]
                code += 1
                k += 1
            code <<= 1


class _Bits:
    def __init__(self, data, pos):
        self.d = data
        self.p = pos
        self.acc = 0
        self.n = 0

    def _fill(self):
        d = self.d
        if self.p >= len(d):
            b = 0
        else:
            b = d[self.p]
            if b == 0xFF:
                nxt = d[self.p + 1] if self.p + 1 < len(d) else 0xD9
                if nxt == 0:
                    self.p += 2
                else:
                    b = 0  # marker: feed zeros, do not advance
            else:
                self.p += 1
        self.acc = (self.acc << 8) | b
        self.n += 8

    def bit(self):
        if self.n == 0:
            self._fill()
        self.n -= 1
        return (self.acc >> self.n) & 1

    def bits(self, k):
        v = 0
        for _ in range(k):
            v = (v << 1) | self.bit()
        return v

    def decode(self, huff):
        code = 0
        for length in range(1, 17):
            code = (code << 1) | self.bit()
            v = huff.lookup.get((length, code))
            if v is not None:
                return v
        raise JpegError("bad Huffman code")

    def restart(self):
        self.acc = 0
        self.n = 0
        d = self.d
        while self.p + 1 < len(d) and not (d[self.p] == 0xFF and 0xD0 <= d[self.p + 1] <= 0xD7):
            self.p += 1
        self.p += 2


def _extend(v, t):
    return v if v >= (1 << (t - 1)) else v - (1 << t) + 1


class Coefficients:
    """Entropy-decoded image: per-component coefficient blocks in natural (row-major) order."""

    def __init__(self):
        self.width = self.height = 0
        self.ncomp = 0
        self.hs = []
        self.vs = []
        self.quant = []      # per component, 64 uint16, natural order
        self.blocks = []     # per component int16 [blocks_h, blocks_w, 8, 8]


def entropy_decode(data):
    """Parse markers and Huffman-decode a baseline (SOF0/SOF1, 8-bit) JPEG."""
    data = bytes(data)
    if len(data) < 4 or data[0] != 0xFF or data[1] != 0xD8:
        raise JpegError("not a JPEG stream")
    qt = {}
    dc = {0: _Huff(*STD_DC_LUMA), 1: _Huff(*STD_DC_CHROMA)}
    ac = {0: _Huff(*STD_AC_LUMA), 1: _Huff(*STD_AC_CHROMA)}
    out = Coefficients()
    comps = []
    restart_interval = 0
    p = 2
    while True:
        while p < len(data) and data[p] != 0xFF:
            p += 1
        while p < len(data) and data[p] == 0xFF:
            p += 1
        if p >= len(data):
            raise JpegError("no scan found")
        m = data[p]
        p += 1
        if m == 0xD9:
            raise JpegError("no scan found")
        if 0xD0 <= m <= 0xD7 or m == 0x01:
            continue
        ln = (data[p] << 8) | data[p + 1]
        seg = data[p + 2:p + ln]
        if m == 0xDB:
            q = 0
            while q < len(seg):
                pq, tq = seg[q] >> 4, seg[q] & 15
                q += 1
                tbl = np.zeros(64, np.uint16)
                for i in range(64):
                    if pq:
                        tbl[ZIGZAG[i]] = (seg[q] << 8) | seg[q + 1]
                        q += 2
                    else:
                        tbl[ZIGZAG[i]] = seg[q]
                        q += 1
                qt[tq] = tbl
        elif m in (0xC0, 0xC1):
            if seg[0] != 8:
                raise JpegError("only 8-bit samples are supported")
            out.height = (seg[1] << 8) | seg[2]
            out.width = (seg[3] << 8) | seg[4]
            out.ncomp = seg[5]
            if out.ncomp not in (1, 3):
                raise JpegError("unsupported number of components")
            for i in range(out.ncomp):
                cid, hv, tq = seg[6 + 3 * i], seg[7 + 3 * i], seg[8 + 3 * i]
                comps.append(dict(id=cid, h=hv >> 4, v=hv & 15, tq=tq))
        elif m in (0xC2, 0xC3, 0xC5, 0xC6, 0xC7, 0xC9, 0xCA, 0xCB, 0xCD, 0xCE, 0xCF):
            raise JpegError("unsupported JPEG process (only baseline sequential Huffman)")
        elif m == 0xC4:
            q = 0
            while q < len(seg):
                tc, th = seg[q] >> 4, seg[q] & 15
                bits = list(seg[q + 1:q + 17])
                n = sum(bits)
                vals = list(seg[q + 17:q + 17 + n])
                q += 17 + n
                (ac if tc else dc)[th] = _Huff(bits, vals)
        elif m == 0xDD:
            restart_interval = (seg[0] << 8) | seg[1]
        elif m == 0xDA:
            ns = seg[0]
            if ns != out.ncomp:
                raise JpegError("non-interleaved scans are not supported")
            for i in range(ns):
                cs, tt = seg[1 + 2 * i], seg[2 + 2 * i]
                c = [c for c in comps if c["id"] == cs][0]
                c["td"], c["ta"] = tt >> 4, tt & 15
            p += ln
            break
        p += ln

    hmax = max(c["h"] for c in comps)
    vmax = max(c["v"] for c in comps)
    if out.ncomp == 1:
        comps[0]["h"] = comps[0]["v"] = 1
        hmax = vmax = 1
    mcux = (out.width + 8 * hmax - 1) // (8 * hmax)
    mcuy = (out.height + 8 * vmax - 1) // (8 * vmax)
    for c in comps:
        out.hs.append(c["h"])
        out.vs.append(c["v"])
        out.quant.append(qt[c["tq"]])
        out.blocks.append(np.zeros((mcuy * c["v"], mcux * c["h"], 64), np.int16))
    br = _Bits(data, p)
    pred = [0] * out.ncomp
    count = 0
    for my in range(mcuy):
        for mx in range(mcux):
            if restart_interval and count and count % restart_interval == 0:
                br.restart()
                pred = [0] * out.ncomp
            count += 1
            for ci, c in enumerate(comps):
                for by in range(c["v"]):
                    for bx in range(c["h"]):
                        blk = out.blocks[ci][my * c["v"] + by, mx * c["h"] + bx]
                        t = br.decode(dc[c["td"]])
                        diff = _extend(br.bits(t), t) if t else 0
                        pred[ci] += diff
                        blk[0] = pred[ci]
                        k = 1
                        while k < 64:
                            rs = br.decode(ac[c["ta"]])
                            r, s = rs >> 4, rs & 15
                            if s == 0:
                                if r != 15:
                                    break
                                k += 16
                                continue
                            k += r
                            if k > 63:
                                raise JpegError("corrupt coefficient run")
                            blk[ZIGZAG[k]] = _extend(br.bits(s), s)
                            k += 1
    out.blocks = [b.reshape(b.shape[0], b.shape[1], 8, 8) for b in out.blocks]
    return out


# ---- inverse DCT -------------------------------------------------------------------------------

CONST_BITS = 13
PASS1_BITS = 2


def _fix(x):
    return int(x * (1 << CONST_BITS) + 0.5)


F_0_298631336 = _fix(0.298631336)
F_0_390180644 = _fix(0.390180644)
F_0_541196100 = _fix(0.541196100)
F_0_765366865 = _fix(0.765366865)
F_0_899976223 = _fix(0.899976223)
F_1_175875602 = _fix(1.175875602)
F_1_501321110 = _fix(1.501321110)
F_1_847759065 = _fix(1.847759065)
F_1_961570560 = _fix(1.961570560)
F_2_053119869 = _fix(2.053119869)
F_2_562915447 = _fix(2.562915447)
F_3_072711026 = _fix(3.072711026)


def _idct_1d(x, shift, first_pass):
    """One 8-point LLM inverse DCT along the last axis of int64 array x -> descaled result."""
    x0, x1, x2, x3, x4, x5, x6, x7 = [x[..., i] for i in range(8)]
    # even part
    z1 = (x2 + x6) * F_0_541196100
    t2 = z1 - x6 * F_1_847759065
    t3 = z1 + x2 * F_0_765366865
    t0 = (x0 + x4) << CONST_BITS
    t1 = (x0 - x4) << CONST_BITS
    e0, e3 = t0 + t3, t0 - t3
    e1, e2 = t1 + t2, t1 - t2
    # odd part
    o0, o1, o2, o3 = x7, x5, x3, x1
    z1 = o0 + o3
    z2 = o1 + o2
    z3 = o0 + o2
    z4 = o1 + o3
    z5 = (z3 + z4) * F_1_175875602
    o0 = o0 * F_0_298631336
    o1 = o1 * F_2_053119869
    o2 = o2 * F_3_072711026
    o3 = o3 * F_1_501321110
    z1 = -z1 * F_0_899976223
    z2 = -z2 * F_2_562915447
    z3 = -z3 * F_1_961570560 + z5
    z4 = -z4 * F_0_390180644 + z5
    o0 += z1 + z3
    o1 += z2 + z4
    o2 += z2 + z3
    o3 += z1 + z4
    rnd = 1 << (shift - 1)
    out = np.stack([e0 + o3, e1 + o2, e2 + o1, e3 + o0, e3 - o0, e2 - o1, e1 - o2, e0 - o3], -1)
    return (out + rnd) >> shift


def idct_blocks(blocks, quant):
    """Dequantise + inverse DCT: int16 [..., 8, 8] coefficient blocks -> uint8 samples [..., 8, 8]."""
    c = blocks.astype(np.int64) * quant.reshape(8, 8).astype(np.int64)
    # pass 1: columns (transform along axis -2), keep PASS1_BITS extra bits
    ws = _idct_1d(np.swapaxes(c, -1, -2), CONST_BITS - PASS1_BITS, True)
    ws = np.swapaxes(ws, -1, -2)
    # pass 2: rows
    out = _idct_1d(ws, CONST_BITS + PASS1_BITS + 3, False)
    return np.clip(out + 128, 0, 255).astype(np.uint8)


def component_plane(blocks, quant):
    s = idct_blocks(blocks, quant)                     # [bh, bw, 8, 8]
    bh, bw = s.shape[:2]
    return s.transpose(0, 2, 1, 3).reshape(bh * 8, bw * 8)


# ---- upsampling and colour conversion --------------------------------------------------------------


def _h2_fancy(row_sum, bias_first, bias_second, shift, scale):
    """Horizontal triangle filter on an array of (possibly vertically pre-summed) rows.

    row_sum[..., x] -> output[..., 2x], output[..., 2x+1] with weights 3:1 towards the nearer
    neighbour; the first and last columns replicate the edge sample.
    """
    s = row_sum.astype(np.int32)
    left = np.concatenate([s[..., :1], s[..., :-1]], -1)
    right = np.concatenate([s[..., 1:], s[..., -1:]], -1)
    even = (s * 3 + left + bias_first) >> shift
    odd = (s * 3 + right + bias_second) >> shift
    # edge columns: the replicated neighbour equals the sample itself, which the formula already gives
    # for scale 4 weights (3*s + s); biases at the edges differ in libjpeg and are patched by the caller.
    out = np.empty(s.shape[:-1] + (s.shape[-1] * 2,), np.int32)
    out[..., 0::2] = even
    out[..., 1::2] = odd
    return out


def upsample_h2v1(plane, out_w):
    """2:1 horizontal fancy upsampling: (3*near + far + {1,2}) >> 2, edges copied."""
    s = plane.astype(np.int32)
    out = _h2_fancy(s, 1, 2, 2, 4)
    out[..., 0] = s[..., 0]
    out[..., -1] = s[..., -1]
    return out[..., :out_w].astype(np.uint8)


def upsample_h2v2(plane, out_w, out_h):
    """2:1 x 2:1 fancy upsampling.

    Vertically each output row is 3*near + far of the two closest input rows (the image
    border replicates the edge row); horizontally the same 3:1 filter is applied to those
    sums with rounding biases 8 (even outputs) and 7 (odd outputs) and a 4-bit shift.
    """
    s = plane.astype(np.int32)
    up = np.concatenate([s[:1], s[:-1]], 0)
    dn = np.concatenate([s[1:], s[-1:]], 0)
    rows = np.empty((s.shape[0] * 2, s.shape[1]), np.int32)
    rows[0::2] = 3 * s + up
    rows[1::2] = 3 * s + dn
    out = _h2_fancy(rows, 8, 7, 4, 16)
    out[:, 0] = (rows[:, 0] * 4 + 8) >> 4
    out[:, -1] = (rows[:, -1] * 4 + 7) >> 4
    return out[:out_h, :out_w].astype(np.uint8)


def _ycc_tables():
    x = np.arange(256, dtype=np.int64) - 128
    one_half = 1 << 15
    fix = lambda v: int(v * 65536 + 0.5)
    cr_r = (fix(1.40200) * x + one_half) >> 16
    cb_b = (fix(1.77200) * x + one_half) >> 16
    cr_g = -fix(0.71414) * x
    cb_g = -fix(0.34414) * x + one_half
    return cr_r, cb_b, cr_g, cb_g


_CR_R, _CB_B, _CR_G, _CB_G = _ycc_tables()


def ycc_to_bgr(y, cb, cr):
    y = y.astype(np.int64)
    r = y + _CR_R[cr]
    g = y + ((_CB_G[cb] + _CR_G[cr]) >> 16)
    b = y + _CB_B[cb]
    return np.clip(np.stack([b, g, r], -1), 0, 255).astype(np.uint8)


def back_end(co):
    """Coefficients -> BGR uint8 image, the way cv::imdecode(IMREAD_COLOR) returns it."""
    w, h = co.width, co.height
    planes = [component_plane(co.blocks[i], co.quant[i]) for i in range(co.ncomp)]
    if co.ncomp == 1:
        g = planes[0][:h, :w]
        return np.stack([g, g, g], -1)
    hmax, vmax = max(co.hs), max(co.vs)
    full = [None] * 3
    for i in range(3):
        fh, fv = hmax // co.hs[i], vmax // co.vs[i]
        cw = (w * co.hs[i] + hmax - 1) // hmax      # downsampled_width
        chh = (h * co.vs[i] + vmax - 1) // vmax
        p = planes[i][:chh, :cw]
        if (fh, fv) == (1, 1):
            full[i] = p[:h, :w]
        elif (fh, fv) == (2, 1):
            full[i] = upsample_h2v1(p, w)[:h]
        elif (fh, fv) == (2, 2):
            full[i] = upsample_h2v2(p, w, h)
        else:
            raise JpegError("unsupported chroma subsampling")
    return ycc_to_bgr(full[0], full[1], full[2])


def decode(data):
    return back_end(entropy_decode(data))
