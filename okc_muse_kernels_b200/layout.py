"""The packed ("stage image") weight format the sm_100a kernels stream, stated in numpy.

The repack is lossless (same number of bytes as the NVFP4 tensors it is made from: 4 bits per
code + one E4M3 byte per 16 codes) and plays the role of the reference's prepare-time repackers
``_pack_weight`` / ``_pack_scales`` / ``_sq_pack`` (muse_moe_w4a16/submission.py:5916-5952), for a
different consumer: here the consumer is one thread per weight row that turns 32 codes into 16
bf16x2 registers and stores them to tensor memory as the A operand of ``tcgen05.mma``.

Geometry
--------
A GEMM ``D[rows, tokens] = W[rows, K] . X[tokens, K]^T`` is cut into *units*: one expert, one pair
of 128-row tiles (gate tile + matching up tile for w13; two adjacent tiles for w2).  A unit is
streamed as K/256 *stages*; a stage is 36 864 contiguous bytes::

    [half 0: K elements 0..127 of the stage, 18 432 B][half 1: K elements 128..255, 18 432 B]
    half       = [tile A part 9 216 B][tile B part 9 216 B]
    tile part  = codes  [chunk c = 0..3][row r = 0..127][16 B]      (8 192 B)
                 scales [chunk c = 0..3][row r = 0..127][ 2 B]      (1 024 B)

so that a whole stage and half a stage are both one contiguous copy (a step with experts of more
than 32 rows streams half stages).

Chunk c of row r holds K elements ``k0 + 32c .. k0 + 32c + 31`` (two 16-element scale blocks): four
32-bit words ``(w0, w1)`` for block 0 and ``(w2, w3)`` for block 1, and the blocks' two scale bytes.

Scale bytes
-----------
A block's E4M3 scale ``2**E * (1 + m/8)`` is kept as the byte ``16 + 8 * (E + 7) + m`` (``SCALE_CODE``;
for a normal E4M3 byte b that is b + 16, the seven subnormals are normalised first).  Shifted left
by four bits it is the exponent and top mantissa bits of a bf16, so one integer multiply-add,
``byte * 0x00100010 + 0x76007600``, yields the bf16x2 ``{scale, scale} * 2**118``.  A scale of zero has
no such code: the repack clears the block's codes instead (every product is zero either way); a
negative scale is folded into the codes' sign bits.

Bits inside a word pair
-----------------------
The 16 codes of a block are bit-permuted so that eight shift-and-mask operations produce eight
bf16x2 registers whose halves are ``code value * 2**-126`` (sign at bit 15, the three magnitude
bits at bits 8:6 of each half): ``out = shift(src) & 0x81C081C0``.  Six registers come straight
from ``w0`` (as is, rotate right 4, shift left 6) and ``w1`` (rotate right 2 and 6, shift left 4);
the bits those leave over in both words are merged with one select,
``u = (w0 & LEFT) | (w1 & ~LEFT)``, and give the last two (rotate right 8, shift left 2).  The left
shifts are multiplies by a power of two, which run on the FMA pipe instead of the busier integer
pipe.  ``PAIR_BITS[j][b]`` is the (word, bit) that holds bit ``b`` of code ``j``.
"""
from __future__ import annotations

import numpy as np

TILE_ROWS = 128
STAGE_K = 256
CHUNK_K = 32
CHUNKS = STAGE_K // CHUNK_K                      # 8
TILE_CODE_BYTES = CHUNKS * TILE_ROWS * 16        # 16384
TILE_SCALE_BYTES = CHUNKS * TILE_ROWS * 2        # 2048
TILE_BYTES = TILE_CODE_BYTES + TILE_SCALE_BYTES  # 18432: one tile's codes and scales of a stage
STAGE_BYTES = 2 * TILE_BYTES                     # 36864
HALF_CHUNKS = CHUNKS // 2                        # 4
HALF_TILE_CODE_BYTES = TILE_CODE_BYTES // 2      # 8192
HALF_TILE_BYTES = TILE_BYTES // 2                # 9216
HALF_STAGE_BYTES = STAGE_BYTES // 2              # 18432

OUT_MASK = 0x81C081C0
# (source, op, amount) of the eight output registers; source 0 = w0, 1 = w1, 2 = u;
# op "r" = rotate right, "l" = shift left (bits shifted out are dropped)
OUT_PLAN = ((0, "r", 0), (0, "r", 4), (0, "l", 6), (1, "r", 2), (1, "r", 6), (1, "l", 4), (2, "r", 8), (2, "l", 2))


def _source_bit(op: str, amount: int, target: int) -> int:
    """Bit of the source word that lands on bit `target` of the shifted word."""
    if op == "r":
        return (target + amount) % 32
    assert target - amount >= 0
    return target - amount
# target bit of code bit b (0 = mantissa, 1..2 = exponent, 3 = sign) in the low half of a register
_HALF_BITS = (6, 7, 8, 15)


def _left_mask() -> int:
    """Bits of w0 that its three rotations do not use (the same residues mod 16 in both halves)."""
    used = 0
    for src, op, amount in OUT_PLAN:
        if src == 0:
            for t in range(32):
                if (OUT_MASK >> t) & 1:
                    used |= 1 << _source_bit(op, amount, t)
    return (~used) & 0xFFFFFFFF


LEFT_MASK = _left_mask()


def _pair_bits():
    table = [[None] * 4 for _ in range(16)]
    seen = set()
    for i, (src, op, amount) in enumerate(OUT_PLAN):
        for half in range(2):
            j = 2 * i + half
            for b in range(4):
                p = _source_bit(op, amount, _HALF_BITS[b] + 16 * half)
                if src == 2:
                    word = 0 if (LEFT_MASK >> p) & 1 else 1
                else:
                    word = src
                assert (word, p) not in seen
                seen.add((word, p))
                table[j][b] = (word, p)
    assert len(seen) == 64
    return table


PAIR_BITS = _pair_bits()
# flat form for the CUDA repack kernel: PAIR_SHIFT[j*4+b] = word*32 + bit
PAIR_SHIFT = [PAIR_BITS[j][b][0] * 32 + PAIR_BITS[j][b][1] for j in range(16) for b in range(4)]


def pack_block(codes16: np.ndarray) -> np.ndarray:
    """uint8 codes [..., 16] (one 16-element scale block) -> uint32 [..., 2] bit-permuted words."""
    c = np.asarray(codes16, dtype=np.uint64)
    out = np.zeros(c.shape[:-1], dtype=np.uint64)
    for j in range(16):
        for b in range(4):
            out |= ((c[..., j] >> np.uint64(b)) & np.uint64(1)) << np.uint64(PAIR_SHIFT[j * 4 + b])
    return np.stack(((out & np.uint64(0xFFFFFFFF)), (out >> np.uint64(32))), axis=-1).astype(np.uint32)


def _rotr(x: np.ndarray, s: int) -> np.ndarray:
    x = x.astype(np.uint32)
    if s == 0:
        return x
    return ((x >> np.uint32(s)) | (x << np.uint32(32 - s))).astype(np.uint32)


def unpack_block_regs(words: np.ndarray) -> np.ndarray:
    """What the device does with a word pair: uint32 [..., 2] -> eight bf16x2 registers [..., 8]
    (before the multiply by the block scale)."""
    w0 = words[..., 0].astype(np.uint32)
    w1 = words[..., 1].astype(np.uint32)
    u = (w0 & np.uint32(LEFT_MASK)) | (w1 & np.uint32(~LEFT_MASK & 0xFFFFFFFF))
    srcs = (w0, w1, u)
    outs = []
    for src, op, amount in OUT_PLAN:
        x = srcs[src]
        x = _rotr(x, amount) if op == "r" else ((x.astype(np.uint64) << np.uint64(amount)) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
        outs.append(x & np.uint32(OUT_MASK))
    return np.stack(outs, axis=-1)


def regs_to_values(regs: np.ndarray) -> np.ndarray:
    """bf16x2 registers [..., 8] -> float32 E2M1 values [..., 16] (undoing the 2**-126)."""
    lo = (regs & np.uint32(0xFFFF)).astype(np.uint32) << np.uint32(16)
    hi = (regs & np.uint32(0xFFFF0000)).astype(np.uint32)
    both = np.stack((lo, hi), axis=-1).reshape(*regs.shape[:-1], 16)
    return (both.view(np.float32).astype(np.float64) * 2.0 ** 126).astype(np.float32)


def _codes(packed: np.ndarray) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8)
    return np.stack((p & 0x0F, p >> 4), axis=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)


def _scale_code_table() -> np.ndarray:
    """E4M3 magnitude bits (0..127) -> the byte kept in the stage image."""
    t = np.zeros(128, dtype=np.uint8)
    t[8:127] = np.arange(8, 127) + 16                 # normal: 2**(b//8 - 7) * (1 + (b%8)/8)
    t[1:8] = (0, 8, 12, 16, 18, 20, 22)               # subnormal b * 2**-9, normalised
    t[0] = 16                                         # zero: the codes are cleared, any finite scale will do
    t[127] = 153                                      # NaN stays NaN
    return t


SCALE_CODE = _scale_code_table()


def scale_code_value(code: np.ndarray) -> np.ndarray:
    """What the device makes of a stored scale byte (undoing the 2**118): float32."""
    pattern = (np.asarray(code, dtype=np.uint32) * np.uint32(16) + np.uint32(0x7600)) << np.uint32(16)
    with np.errstate(invalid="ignore"):
        return (pattern.view(np.float32).astype(np.float64) * 2.0 ** -118).astype(np.float32)


def pack_tile_stage(packed_rows: np.ndarray, sf_rows: np.ndarray) -> np.ndarray:
    """One tile's codes [chunk][row][16 B] and scales [chunk][row][2 B] of a stage, chunk-major, before
    they are dealt into the two halves of the stage image: packed codes uint8 [128, 128] (K = 256) +
    scales uint8 [128, 16] -> uint8 [18432]."""
    codes = _codes(packed_rows).reshape(TILE_ROWS, CHUNKS, 2, 16)         # row, chunk, block, code
    sc = np.asarray(sf_rows, dtype=np.uint8).reshape(TILE_ROWS, CHUNKS, 2)
    mag = sc & 0x7F
    codes = np.where((mag == 0)[..., None], 0, codes)                      # zero scale: clear the codes
    codes = np.where((sc & 0x80 != 0)[..., None], codes ^ 8, codes)        # negative scale: flip the signs
    words = pack_block(codes)                                              # row, chunk, block, 2
    code_img = np.ascontiguousarray(words.transpose(1, 0, 2, 3)).view(np.uint8).reshape(-1)
    scale_img = np.ascontiguousarray(SCALE_CODE[mag].transpose(1, 0, 2)).reshape(-1)
    return np.concatenate((code_img, scale_img))


def repack_matrix(packed: np.ndarray, sf: np.ndarray, pair_rows) -> np.ndarray:
    """Repack one expert's matrix (packed uint8 [rows, K/2], sf uint8 [rows, K/16]).

    ``pair_rows(p) -> (first row of tile A, first row of tile B)``.  Returns uint8
    [n_pairs, K/256, 36864]."""
    rows, kb = packed.shape
    k = kb * 2
    n_pairs = rows // (2 * TILE_ROWS)
    stages = k // STAGE_K
    out = np.empty((n_pairs, stages, STAGE_BYTES), dtype=np.uint8)
    for p in range(n_pairs):
        ra, rb = pair_rows(p)
        for s in range(stages):
            for t, r0 in enumerate((ra, rb)):
                tile = pack_tile_stage(packed[r0:r0 + TILE_ROWS, s * 128:(s + 1) * 128],
                                       sf[r0:r0 + TILE_ROWS, s * 16:(s + 1) * 16])
                codes = tile[:TILE_CODE_BYTES].reshape(2, HALF_TILE_CODE_BYTES)        # chunks 0..3 | 4..7
                scales = tile[TILE_CODE_BYTES:].reshape(2, TILE_SCALE_BYTES // 2)
                for h in range(2):
                    o = h * HALF_STAGE_BYTES + t * HALF_TILE_BYTES
                    out[p, s, o:o + HALF_TILE_CODE_BYTES] = codes[h]
                    out[p, s, o + HALF_TILE_CODE_BYTES:o + HALF_TILE_BYTES] = scales[h]
    return out


def repack_w13(packed: np.ndarray, sf: np.ndarray) -> np.ndarray:
    """w13 of one expert ([2I, H/2], rows [0,I) gate, [I,2I) up): pair p = gate rows 128p.. with
    up rows I + 128p.. ."""
    inter = packed.shape[0] // 2
    return repack_matrix(packed, sf, lambda p: (TILE_ROWS * p, inter + TILE_ROWS * p))


def repack_w2(packed: np.ndarray, sf: np.ndarray) -> np.ndarray:
    """w2 of one expert ([H, I/2]): pair p = rows 256p.. and 256p + 128.. ."""
    return repack_matrix(packed, sf, lambda p: (2 * TILE_ROWS * p, 2 * TILE_ROWS * p + TILE_ROWS))


def packed_bytes(hidden: int, inter: int) -> tuple[int, int]:
    """Bytes of one expert's repacked w13 and w2."""
    b13 = (inter // TILE_ROWS) * (hidden // STAGE_K) * STAGE_BYTES
    b2 = (hidden // (2 * TILE_ROWS)) * (inter // STAGE_K) * STAGE_BYTES
    return b13, b2
