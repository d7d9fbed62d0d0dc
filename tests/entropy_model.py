"""Model of the bookkeeping of the block-parallel JPEG entropy kernel (aeon_b200/csrc/jpeg_entropy.cu): segments, guessed
entry states, checkpoints, rounds of re-decoding with an early exit at a checkpoint passed in a noted state, block counts,
and the storing pass dealt out in pieces between checkpoints.  Plain python over the bit string of a baseline JPEG; the
kernel follows the same steps.  `simulate` returns what the kernel would count and every inconsistency it finds: a segment
whose block count differs from the true one, a piece that would start at a wrong block number or meet an invalid symbol, a
checkpoint the storing pass needs that no run has written.  Test infrastructure only."""
import numpy as np

from oracle import jpeg as J

NCHECK = 3           # checkpoints inside a segment
MIN_SEGMENT = 160    # bytes


def _parse(blob):
    """Huffman tables, sampling factors, table selectors, picture size and the offset of the entropy-coded data."""
    dc = {0: J._Huff(*J.STD_DC_LUMA), 1: J._Huff(*J.STD_DC_CHROMA)}
    ac = {0: J._Huff(*J.STD_AC_LUMA), 1: J._Huff(*J.STD_AC_CHROMA)}
    comps, width, height, p = [], 0, 0, 2
    while True:
        assert blob[p] == 0xFF
        marker = blob[p + 1]
        p += 2
        length = (blob[p] << 8) | blob[p + 1]
        seg = blob[p + 2:p + length]
        if marker == 0xC4:
            q = 0
            while q < len(seg):
                tc, th = seg[q] >> 4, seg[q] & 15
                bits = list(seg[q + 1:q + 17])
                vals = list(seg[q + 17:q + 17 + sum(bits)])
                q += 17 + sum(bits)
                (ac if tc else dc)[th] = J._Huff(bits, vals)
        elif marker == 0xC0:
            height, width = (seg[1] << 8) | seg[2], (seg[3] << 8) | seg[4]
            comps = [(seg[7 + 3 * i] >> 4, seg[7 + 3 * i] & 15) for i in range(seg[5])]
        elif marker == 0xDA:
            selectors = [(seg[2 + 2 * i] >> 4, seg[2 + 2 * i] & 15) for i in range(seg[0])]
            return p + length, dc, ac, comps, selectors, width, height
        p += length


def simulate(blob, threads=512, checkpoint_past_end=False):
    """Runs the kernel's passes over one stream.  `checkpoint_past_end` restores the rule that once let a run note (or fall
    into step at) a checkpoint lying within a symbol's reach past the end of the last segment."""
    start, dc, ac, comps, selectors, width, height = _parse(blob)
    scan = blob[start:-2]
    clean, i = bytearray(), 0
    while i < len(scan):                                   # the copy without stuffed bytes
        clean.append(scan[i])
        i += 2 if scan[i] == 0xFF and i + 1 < len(scan) and scan[i + 1] == 0 else 1
    total_bit = len(clean) * 8
    bits = np.unpackbits(np.frombuffer(bytes(clean) + b"\0" * 8, np.uint8)).tolist()

    hmax, vmax = max(c[0] for c in comps), max(c[1] for c in comps)
    block_comp = []                                        # component of every block of an MCU
    for ci, (h, v) in enumerate(comps):
        block_comp += [ci] * (h * v if len(comps) > 1 else 1)
    bpm = len(block_comp)
    mcux = -(-width // (8 * hmax)) if len(comps) > 1 else -(-width // 8)
    mcuy = -(-height // (8 * vmax)) if len(comps) > 1 else -(-height // 8)
    total_blocks = mcux * mcuy * bpm

    def symbol(p, b, k):
        """(bits taken, value bits, advance of the zig-zag index) of the symbol at bit p in state (b, k)."""
        table = dc[selectors[block_comp[b]][0]] if k == 0 else ac[selectors[block_comp[b]][1]]
        code = 0
        for length in range(1, 17):
            code = (code << 1) | bits[p + length - 1]
            sym = table.lookup.get((length, code))
            if sym is not None:
                size, run = sym & 15, sym >> 4
                if k == 0:
                    return length + size, size, 1 if run == 0 else 127
                return length + size, size, (run + 1) if size else (16 if run == 15 else 64)
        return 16, 0, 127                                  # invalid code

    block_ends, p, b, k, done = [], 0, 0, 0, 0             # the true decoder: where every block's last symbol starts
    while done < total_blocks:
        taken, _, advance = symbol(p, b, k)
        assert advance != 127
        if k + advance >= 64:
            block_ends.append(p)
        p, k = p + taken, k + advance
        if k >= 64:
            k, done, b = 0, done + 1, (b + 1) % bpm
    block_ends = np.array(block_ends)

    seg = max((-(-len(clean) // threads) + 3) & ~3, MIN_SEGMENT)
    nseg = -(-len(clean) // seg)
    step = seg * 8 // (NCHECK + 1)

    def run(p, b, k, pend, notes, compare, old_blocks, storing=False):
        blocks, bad, merged, j = 0, False, False, 0
        check_at = None
        if not storing and (checkpoint_past_end or notes["first"] < pend):
            check_at = notes["first"]
        while p < pend:
            taken, size, advance = symbol(p, b, k)
            if storing and (advance == 127 or (k != 0 and size and k + advance - 1 > 63)):
                bad = True
            p, k = p + taken, k + advance
            if k >= 64:
                k, blocks, b = 0, blocks + 1, (b + 1) % bpm
            if check_at is not None and p >= check_at:
                assert p - check_at <= 30
                key = (p - check_at) << 10 | b << 6 | k
                if compare and notes["key"][j] == key:     # in step with the remembered run
                    was = notes["blocks"][j]
                    for later in range(j, NCHECK):
                        if notes["blocks"][later] is not None:
                            notes["blocks"][later] += blocks - was
                    blocks += old_blocks - was
                    merged = True
                    break
                notes["key"][j], notes["blocks"][j] = key, blocks
                j += 1
                more = j < NCHECK and (checkpoint_past_end or check_at + step < pend)
                check_at = check_at + step if more else None
        return p, b, k, blocks, bad, merged

    segments = []
    for t in range(nseg):                                  # first pass: guessed entry states
        first, last = t * seg * 8, min(total_bit, (t + 1) * seg * 8)
        notes = {"first": first + step, "key": [None] * NCHECK, "blocks": [None] * NCHECK}
        p, b, k, blocks, _, _ = run(first, 0, 0, last, notes, False, 0)
        segments.append({"first": first, "last": last, "notes": notes, "entry": (first, 0, 0), "exit": (p, b, k), "count": blocks})
    rounds = 0
    while True:                                            # rounds: the left neighbour's exit state is the entry state
        rounds += 1
        candidates = [None] + [segments[t - 1]["exit"] for t in range(1, nseg)]
        again = False
        for t in range(1, nseg):
            s = segments[t]
            if candidates[t] != s["entry"]:
                again = True
                p, b, k, blocks, _, merged = run(*candidates[t], s["last"], s["notes"], True, s["count"])
                s["entry"], s["count"] = candidates[t], blocks
                if not merged:
                    s["exit"] = (p, b, k)
        if not again:
            break
        assert rounds <= nseg

    problems = []
    counted = sum(s["count"] for s in segments)
    if counted != total_blocks:
        problems.append(("counted", counted, total_blocks))
    first_block = 0
    for t, s in enumerate(segments):                       # the storing pass, piece by piece
        true_count = int(((block_ends >= s["entry"][0]) & (block_ends < s["last"])).sum())
        if true_count != s["count"]:
            problems.append(("segment count", t, s["count"], true_count))
        for piece in range(NCHECK + 1):
            at = s["first"] + piece * step
            if at >= s["last"]:
                continue
            if piece == 0:
                (p0, b0, k0), before = s["entry"], 0
            else:
                key = s["notes"]["key"][piece - 1]
                if key is None:
                    problems.append(("unwritten checkpoint", t, piece))
                    continue
                p0, b0, k0, before = at + (key >> 10), key >> 6 & 15, key & 63, s["notes"]["blocks"][piece - 1]
            if p0 < total_bit and int((block_ends < p0).sum()) != first_block + before:
                problems.append(("piece block number", t, piece))
            if run(p0, b0, k0, min(s["last"], at + step), None, False, 0, storing=True)[4]:
                problems.append(("piece meets an invalid symbol", t, piece))
        first_block += s["count"]
    return {"bytes": len(clean), "segment": seg, "segments": nseg, "rounds": rounds, "counted": counted,
            "total_blocks": total_blocks, "problems": problems}
