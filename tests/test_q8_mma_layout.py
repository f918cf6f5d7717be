"""The index arithmetic of the Q8_0 tensor-core form (csrc/gemv_q8_mma.cu) replayed on the CPU: shared-memory layout of a
stage (rows 1104 bytes apart), byte offsets and byte permutes of the A fragments for even and odd blocks, the entries'
codes and deltas of the B fragments and accumulator cells, the ownership of lane classes by warps, the swizzled class-sum
scratch and the butterfly per row - emulated with the documented fragment layout of mma.sync.m16n8k32 (A row = lane / 4
and + 8, k bytes 4 (lane % 4) and + 16; B column = lane / 4; C cells (lane / 4 [+ 8], 2 (lane % 4) [+ 1])) - must give the
oracle's Q8_0 x A8 products bit for bit. No GPU: this guards the layout reasoning, the GPU parity tests guard the kernel."""
import numpy as np

PITCH, RUN_BYTES, BLOCK = 1104, 1088, 34


def _word(buf, off):
    return int.from_bytes(bytes(buf[off:off + 4]), "little")


def _prmt5432(a, b):          # bytes 2, 3 of a then bytes 0, 1 of b
    return ((a >> 16) & 0xFFFF) | ((b & 0xFFFF) << 16)


def _s8x4(w):
    return np.frombuffer(int(w).to_bytes(4, "little"), np.int8).astype(np.int64)


def _butterfly(v):
    v = v.astype(np.float32).copy()
    d = 16
    while d:
        v = np.array([np.float32(v[l]) + np.float32(v[l ^ d]) for l in range(32)], np.float32)
        d >>= 1
    return v[0]


def emulate_tile(wbytes, codes, deltas, groups):
    """wbytes [16][groups * 34] uint8, codes [8][K] int8, deltas [8][groups] -> products [16][8] as the kernel forms them."""
    nruns = (groups + 31) // 32
    boxes = []
    for run in range(nruns):                       # one tiled copy per run: 1104 bytes per row, zero filled past the row
        box = np.zeros((16, PITCH), np.uint8)
        lo = run * RUN_BYTES
        hi = min(lo + PITCH, wbytes.shape[1])
        box[:, :hi - lo] = wbytes[:, lo:hi]
        boxes.append(box)
    K = codes.shape[1]
    xc = np.zeros((8, K + 16), np.uint8)           # the entries' codes lie K + 16 bytes apart
    xc[:, :K] = codes.view(np.uint8)
    cls = np.zeros(16 * 8 * 32, np.float32)
    for warp in range(16):
        acc = np.zeros((2, 32, 4), np.float32)
        for run in range(nruns):
            for c in range(2):
                b = run * 32 + 2 * warp + c
                if b >= groups:
                    continue
                blk = BLOCK * (2 * warp + c)
                A = np.zeros((16, 32), np.int64)
                B = np.zeros((32, 8), np.int64)
                for lane in range(32):
                    gid, t4 = lane >> 2, lane & 3
                    ra, rb = boxes[run][gid], boxes[run][gid + 8]
                    if c == 1:                     # odd block of the run: quants on a word
                        a0, a2 = _word(ra, blk + 2 + 4 * t4), _word(ra, blk + 2 + 4 * t4 + 16)
                        a1, a3 = _word(rb, blk + 2 + 4 * t4), _word(rb, blk + 2 + 4 * t4 + 16)
                    else:                          # even block: quants start in the upper half of a word
                        a0 = _prmt5432(_word(ra, blk + 4 * t4), _word(ra, blk + 4 * t4 + 4))
                        a2 = _prmt5432(_word(ra, blk + 4 * t4 + 16), _word(ra, blk + 4 * t4 + 20))
                        a1 = _prmt5432(_word(rb, blk + 4 * t4), _word(rb, blk + 4 * t4 + 4))
                        a3 = _prmt5432(_word(rb, blk + 4 * t4 + 16), _word(rb, blk + 4 * t4 + 20))
                    b0, b1 = _word(xc[gid], 4 * t4 + 32 * b), _word(xc[gid], 4 * t4 + 32 * b + 16)
                    A[gid, 4 * t4:4 * t4 + 4], A[gid + 8, 4 * t4:4 * t4 + 4] = _s8x4(a0), _s8x4(a1)
                    A[gid, 16 + 4 * t4:20 + 4 * t4], A[gid + 8, 16 + 4 * t4:20 + 4 * t4] = _s8x4(a2), _s8x4(a3)
                    B[4 * t4:4 * t4 + 4, gid], B[16 + 4 * t4:20 + 4 * t4, gid] = _s8x4(b0), _s8x4(b1)
                Cm = A @ B
                for lane in range(32):
                    gid, t4 = lane >> 2, lane & 3
                    sa = np.float32(np.frombuffer(bytes(boxes[run][gid][blk:blk + 2]), np.float16)[0])
                    sb = np.float32(np.frombuffer(bytes(boxes[run][gid + 8][blk:blk + 2]), np.float16)[0])
                    d0, d1 = deltas[2 * t4, b], deltas[2 * t4 + 1, b]
                    cells = (Cm[gid, 2 * t4], Cm[gid, 2 * t4 + 1], Cm[gid + 8, 2 * t4], Cm[gid + 8, 2 * t4 + 1])
                    sds = (np.float32(sa * d0), np.float32(sa * d1), np.float32(sb * d0), np.float32(sb * d1))
                    for i in range(4):
                        acc[c, lane, i] = np.float32(acc[c, lane, i] + np.float32(np.float32(cells[i]) * sds[i]))
        for c in range(2):
            for lane in range(32):
                gid, t4 = lane >> 2, lane & 3
                for i in range(4):
                    pair = (gid + 8 * (i >> 1)) * 8 + 2 * t4 + (i & 1)
                    cls[pair * 32 + ((2 * warp + c + pair) & 31)] = acc[c, lane, i]
    out = np.zeros((16, 8), np.float32)
    for warp in range(16):                         # warp w folds row w: lane = class
        for i in range(8):
            pair = warp * 8 + i
            out[warp, i] = _butterfly(np.array([cls[pair * 32 + ((lane + pair) & 31)] for lane in range(32)], np.float32))
    return out


def test_fragment_layout_gives_the_contract_bits(oracle):
    rng = np.random.default_rng(5)
    for K in (1024, 1280, 2304):                   # whole runs, and a last run of 8 blocks
        groups = K // 32
        scale = rng.uniform(0.01, 0.1, (16, groups)).astype(np.float16)
        q = rng.integers(-127, 128, (16, groups, 32)).astype(np.int8)
        w = np.zeros((16, groups * BLOCK), np.uint8)
        for g in range(groups):
            w[:, BLOCK * g:BLOCK * g + 2] = scale[:, g:g + 1].view(np.uint8)
            w[:, BLOCK * g + 2:BLOCK * g + BLOCK] = q[:, g].view(np.uint8)
        codes = rng.integers(-127, 128, (8, K)).astype(np.int8)
        deltas = rng.uniform(0.001, 0.01, (8, groups)).astype(np.float32)
        want = oracle.gemv_q8_0_a8(w, K, codes, deltas)          # [entries][rows]
        got = emulate_tile(w, codes, deltas, groups)             # [rows][entries]
        assert np.array_equal(got.T.copy().view(np.uint32), want.view(np.uint32)), K
