"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark configurations.

The reference measures this path on private GGUF model files or on synthetic blocks; nothing public ships with it, so
every tensor here is drawn from a seeded numpy generator. Blocks are written in the exact GGUF byte layout the kernels
consume:
  Q8_0 block (34 B):        fp16 d (little endian) | int8 q[32]
  Q4_K super-block (144 B): fp16 d | fp16 dmin | 12 B of packed 6-bit (scale, min) x 8 | 128 B of 4-bit quants
  Q5_K super-block (176 B): as Q4_K with 32 B of high bits between the packed factors and the nibbles
  Q5_1 block (24 B):        fp16 d | fp16 m | 32 high bits | 16 B of 4-bit quants
"""
import numpy as np

Q8_0_BLOCK = 34
Q4_K_BLOCK = 144
Q5_K_BLOCK = 176
Q5_1_BLOCK = 24
Q2_K_BLOCK = 84


def q8_0_blocks(rng, nblocks, scale=0.01):
    """d = fp16(|N(0,1)| * scale), quants uniform in [-127, 127]."""
    out = np.empty((nblocks, Q8_0_BLOCK), np.uint8)
    d = (np.abs(rng.standard_normal(nblocks, dtype=np.float32)) * scale).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(nblocks, 2)
    out[:, 2:] = rng.integers(-127, 128, size=(nblocks, 32), dtype=np.int8).view(np.uint8)
    return out


def q4_k_blocks(rng, nblocks, scale=0.01 / 32):
    """d, dmin = fp16(|N(0,1)| * scale); the eight 6-bit sub-scales and mins uniform in 0..63 (every packing of
    twelve uniform bytes is such a draw); 256 nibbles uniform in 0..15."""
    out = rng.integers(0, 256, size=(nblocks, Q4_K_BLOCK), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((nblocks, 2), dtype=np.float32)) * scale).astype(np.float16)
    out[:, 0:4] = dd.view(np.uint8).reshape(nblocks, 4)
    return out


def q5_k_blocks(rng, nblocks, scale=0.01 / 64):
    """As q4_k_blocks with 5-bit quants: every byte but the two fp16 factors uniform."""
    out = rng.integers(0, 256, size=(nblocks, Q5_K_BLOCK), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((nblocks, 2), dtype=np.float32)) * scale).astype(np.float16)
    out[:, 0:4] = dd.view(np.uint8).reshape(nblocks, 4)
    return out


def q2_k_blocks(rng, nblocks, scale=0.01 / 8):
    """84-byte super-blocks: 16 bytes of (4-bit scale | 4-bit min << 4), 64 bytes of 2-bit quants, fp16 d, fp16 dmin
    (d, dmin = fp16(|N(0,1)| * scale)); every byte but the two factors uniform."""
    out = rng.integers(0, 256, size=(nblocks, Q2_K_BLOCK), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((nblocks, 2), dtype=np.float32)) * scale).astype(np.float16)
    out[:, 80:84] = dd.view(np.uint8).reshape(nblocks, 4)
    return out


def q5_1_blocks(rng, nblocks, scale=0.01 / 16):
    """d = fp16(|N(0,1)| * scale), m = fp16(N(0,1) * scale * 8), 5-bit quants uniform in 0..31."""
    out = rng.integers(0, 256, size=(nblocks, Q5_1_BLOCK), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(nblocks, dtype=np.float32)) * scale).astype(np.float16)
    m = (rng.standard_normal(nblocks, dtype=np.float32) * scale * 8).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(nblocks, 2)
    out[:, 2:4] = m.view(np.uint8).reshape(nblocks, 2)
    return out


def pack_q4k_factors(scales, mins):
    """Twelve bytes holding eight (scale, min) 6-bit pairs, the get_scale_min_k4 packing."""
    b = np.zeros(12, np.uint8)
    for j in range(8):
        s, m = int(scales[j]), int(mins[j])
        if j < 4:
            b[j] |= s & 63
            b[j + 4] |= m & 63
        else:
            b[j + 4] |= (s & 15) | ((m & 15) << 4)
            b[j - 4] |= (s >> 4) << 6
            b[j] |= (m >> 4) << 6
    return b


def row_bytes(ggml_type, width):
    return {7: width // 32 * Q5_1_BLOCK, 8: width // 32 * Q8_0_BLOCK, 10: width // 256 * Q2_K_BLOCK, 13: width // 256 * Q5_K_BLOCK}.get(ggml_type, width // 256 * Q4_K_BLOCK)


def expert_tensors(rng, experts, hidden, inter, gate_type, down_type):
    """gate, up [experts][inter][hidden / B] and down [experts][hidden][inter / B] as flat uint8 arrays."""
    def tensor(t, rows, width):
        if t == 8:
            return q8_0_blocks(rng, experts * rows * (width // 32)).reshape(-1)
        if t == 7:
            return q5_1_blocks(rng, experts * rows * (width // 32)).reshape(-1)
        if t == 10:
            return q2_k_blocks(rng, experts * rows * (width // 256)).reshape(-1)
        if t == 13:
            return q5_k_blocks(rng, experts * rows * (width // 256)).reshape(-1)
        return q4_k_blocks(rng, experts * rows * (width // 256)).reshape(-1)
    return tensor(gate_type, inter, hidden), tensor(gate_type, inter, hidden), tensor(down_type, hidden, inter)


def router_weight(rng, experts, hidden, std=0.02):
    return (rng.standard_normal((experts, hidden), dtype=np.float32) * np.float32(std)).astype(np.float32)


def activations(rng, rows, hidden, bf16=False):
    x = rng.standard_normal((rows, hidden), dtype=np.float32)
    if bf16:
        x = bf16_round(x)
    return x


def bf16_round(x):
    """Round FP32 to the nearest bfloat16 (ties to even), returned as FP32."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def bf16_bits(x):
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def zipf_logit_bias(rng, experts, s=1.1):
    """log of a Zipf(s) pmf over a seeded permutation of the experts: added to the router logits it skews the load."""
    rank = rng.permutation(experts).astype(np.float64) + 1.0
    pmf = rank ** (-s)
    pmf /= pmf.sum()
    return np.log(pmf).astype(np.float32)
