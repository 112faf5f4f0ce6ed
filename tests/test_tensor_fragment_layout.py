"""The lane / byte bookkeeping of the tensor-core evaluation kernels (project_b200/csrc/eval.cu), restated with integers:
mma.sync m16n8k32 (u8 x u8 -> s32) is emulated from its fragment layout, the operands are loaded and transposed the way
the kernels do it, and the folded 17-limb sums must equal the exact integer inner products.  Runs without a GPU; the
kernels themselves are compared with the oracle in the GPU tests."""
import numpy as np

R = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001


def prmt(x, y, sel):
    b = [(x >> (8 * i)) & 255 for i in range(4)] + [(y >> (8 * i)) & 255 for i in range(4)]
    return sum(b[(sel >> (4 * i)) & 7] << (8 * i) for i in range(4))


def transpose4(x):
    """four words (one per row) -> four words (one per byte index), as load_rows_transposed does"""
    t0, t1 = prmt(x[0], x[1], 0x5140), prmt(x[2], x[3], 0x5140)
    t2, t3 = prmt(x[0], x[1], 0x7362), prmt(x[2], x[3], 0x7362)
    return [prmt(t0, t1, 0x5410), prmt(t0, t1, 0x7632), prmt(t2, t3, 0x5410), prmt(t2, t3, 0x7632)]


def mma(c, a, b):
    """c[lane][4] += A (16 x 32) * B (32 x 8) with the PTX fragment layout of m16n8k32 for 8-bit operands"""
    A = np.zeros((16, 32), dtype=np.int64)
    B = np.zeros((32, 8), dtype=np.int64)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for i in range(16):
            row = g if (i < 4 or 8 <= i < 12) else g + 8
            col = t * 4 + (i & 3) + (16 if i >= 8 else 0)
            A[row, col] = (a[lane][i // 4] >> (8 * (i % 4))) & 255
        for i in range(8):
            B[t * 4 + (i & 3) + (16 if i >= 4 else 0), g] = (b[lane][i // 4] >> (8 * (i % 4))) & 255
    C = A @ B
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for i in range(4):
            c[lane][i] += int(C[g if i < 2 else g + 8, t * 2 + (i & 1)])


def word_of(rows, row, g):
    return int(sum(int(rows[row, 4 * g + j]) << (8 * j) for j in range(4)))


def to_int(row):
    return sum(int(v) << (8 * i) for i, v in enumerate(row))


def test_field_element_columns():
    rng = np.random.default_rng(1)
    rows_here = 45  # a ragged chunk: the rows behind it count as zero
    W = rng.integers(0, 256, size=(64, 32), dtype=np.int64)
    F = rng.integers(0, 256, size=(64, 32), dtype=np.int64)
    c = [[[[0] * 4 for _ in range(4)] for _ in range(2)] for _ in range(32)]
    for step in range(2):
        fbs, was = [], []
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            fb, wa = [], []
            for h in range(2):
                f = transpose4([word_of(F, step * 32 + 16 * h + t + 4 * q, g) for q in range(4)])
                keep = sum(0xFF << (8 * q) for q in range(4) if step * 32 + 16 * h + t + 4 * q < rows_here)
                fb.append([v & keep for v in f])
                wa.append(transpose4([word_of(W, step * 32 + 16 * h + t + 4 * q, g) for q in range(4)]))
            fbs.append(fb)
            was.append(wa)
        for mt in range(2):
            a = [[was[l][0][2 * mt], was[l][0][2 * mt + 1], was[l][1][2 * mt], was[l][1][2 * mt + 1]] for l in range(32)]
            for nt in range(4):
                mma([c[l][mt][nt] for l in range(32)], a, [[fbs[l][0][nt], fbs[l][1][nt]] for l in range(32)])
    matrix = [0] * 1024
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for mt in range(2):
            for nt in range(4):
                for i in range(4):
                    matrix[(4 * g + 2 * mt + (i >> 1)) * 32 + 8 * t + 4 * (i & 1) + nt] = c[lane][mt][nt][i]
    diagonal = [0] * 64
    for lane in range(32):
        for a_ in range(32):
            diagonal[lane + (32 if a_ > lane else 0)] += matrix[31 * a_ + lane + (32 if a_ > lane else 0)]
    limbs = [diagonal[4 * j] + (diagonal[4 * j + 1] << 8) + (diagonal[4 * j + 2] << 16) + (diagonal[4 * j + 3] << 24) for j in range(16)]
    assert sum(v << (32 * j) for j, v in enumerate(limbs)) == sum(to_int(W[i]) * to_int(F[i]) for i in range(rows_here))


def test_groups_of_integer_columns():
    rng = np.random.default_rng(5)
    rows = 50
    W = rng.integers(0, 256, size=(64, 32), dtype=np.int64)
    values = [[int(rng.integers(-(1 << 40), 1 << 40)) for _ in range(64)] for _ in range(3)] + [[int(rng.integers(0, 1 << 32)) for _ in range(64)]]
    values[0][:3] = [-(1 << 63), (1 << 63) - 1, -1]
    wide = [True, True, True, False]  # three I64 columns and a U32 column

    def value_word(col, row, which):
        if row >= rows:
            return 0
        if wide[col]:
            return ((values[col][row] & (2**64 - 1)) >> (32 * which)) & 0xFFFFFFFF
        return values[col][row] if which == 0 else 0

    cv = [[[[0] * 4 for _ in range(4)] for _ in range(2)] for _ in range(32)]
    cs = [[[0] * 4 for _ in range(2)] for _ in range(32)]
    for step in range(2):
        fbs, sbs, was = [], [], []
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            col, which = g >> 1, g & 1
            fb, sb, wa = [], [], []
            for h in range(2):
                f = transpose4([value_word(col, step * 32 + 16 * h + t + 4 * q, which) for q in range(4)])
                fb.append(f)
                sb.append(((f[3] >> 7) & 0x01010101) if (wide[col] and which == 1) else 0)
                wa.append(transpose4([word_of(W, r, g) if (r := step * 32 + 16 * h + t + 4 * q) < rows else 0 for q in range(4)]))
            fbs.append(fb)
            sbs.append(sb)
            was.append(wa)
        for mt in range(2):
            a = [[was[l][0][2 * mt], was[l][0][2 * mt + 1], was[l][1][2 * mt], was[l][1][2 * mt + 1]] for l in range(32)]
            for nt in range(4):
                mma([cv[l][mt][nt] for l in range(32)], a, [[fbs[l][0][nt], fbs[l][1][nt]] for l in range(32)])
            mma([cs[l][mt] for l in range(32)], a, [[sbs[l][0], sbs[l][1]] for l in range(32)])
    stride = 37
    matrix = [0] * (32 * stride)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for mt in range(2):
            for i in range(4):
                a_, n = 4 * g + 2 * mt + (i >> 1), 2 * t + (i & 1)
                for nt in range(4):
                    matrix[a_ * stride + (n >> 1) * 8 + 4 * (n & 1) + nt] = cv[lane][mt][nt][i]
                if n & 1:
                    matrix[a_ * stride + 32 + (n >> 1)] = cs[lane][mt][i]
    for col in range(4):
        diagonal = [sum(matrix[(d - b) * stride + col * 8 + b] for b in range(8) if 0 <= d - b < 32) for d in range(40)]
        value = sum((diagonal[4 * j] + (diagonal[4 * j + 1] << 8) + (diagonal[4 * j + 2] << 16) + (diagonal[4 * j + 3] << 24)) << (32 * j) for j in range(10))
        negative = sum(sum(matrix[(4 * j + q) * stride + 32 + col] << (8 * q) for q in range(4)) << (32 * (j + 2)) for j in range(8))
        total = value + (R << 84) - negative
        want = sum(to_int(W[i]) * values[col][i] for i in range(rows))
        assert 0 <= total < 2**544 and total - want == R << 84


def test_row_wise_linear_form():
    """linear_form_tensor_kernel: the words of a matrix row are the A fragments as they lie in memory (upper halves of the
    entries with their top bit flipped: u = v + 2^63), the powers enter as the byte table P(8j + b) = p_j 2^(8b) mod r in
    B-fragment order, and a quad of lanes adds the 32 byte sums of a row."""
    rng = np.random.default_rng(9)
    cols, rows = 8, 32  # two contraction steps of 32 bytes
    values = rng.integers(-(1 << 62), 1 << 62, size=(rows, cols), dtype=np.int64)
    values[0, :3] = [np.iinfo(np.int64).min, np.iinfo(np.int64).max, -1]
    powers = [int.from_bytes(rng.bytes(32), "little") % R for _ in range(cols)]
    # the table, written the way linear_form_table_kernel writes it
    table = bytearray(cols * 256)
    for kappa in range(cols * 8):
        entry = (powers[kappa >> 3] << (8 * (kappa & 7))) % R
        step, within = kappa >> 5, kappa & 31
        h, t, q = within >> 4, (within & 15) >> 2, within & 3
        for n in range(32):
            word = ((step * 4 + (n >> 3)) * 2 + h) * 32 + (n & 7) * 4 + t
            table[word * 4 + q] = (entry >> (8 * n)) & 255
    words = np.frombuffer(bytes(table), dtype="<u4")
    row_bytes = [int(v) & (2**64 - 1) for v in values.reshape(-1)]

    def row_word(r, byte_offset):
        entry = row_bytes[r * cols + byte_offset // 8]
        return (entry >> (8 * (byte_offset % 8))) & 0xFFFFFFFF

    c = [[[[0] * 4 for _ in range(4)] for _ in range(2)] for _ in range(32)]
    for s in range(cols // 4):
        for mt in range(2):
            a = []
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                flip = 0x80000000 if t & 1 else 0
                a.append([row_word(16 * mt + 8 * half + g, 32 * s + 16 * k16 + 4 * t) ^ flip for k16 in range(2) for half in range(2)])
            for nt in range(4):
                b = [[int(words[s * 256 + (nt * 2 + h) * 32 + lane]) for h in range(2)] for lane in range(32)]
                mma([c[l][mt][nt] for l in range(32)], a, b)
    bias = ((1 << 63) * sum(powers)) % R
    for mt in range(2):
        for half in range(2):
            for g in range(8):
                total = 0
                for t in range(4):  # the quad of lanes that shares the row
                    lane = 4 * g + t
                    for nt in range(4):
                        v = c[lane][mt][nt][2 * half] + (c[lane][mt][nt][2 * half + 1] << 8)
                        total += (v << (16 * t)) << (64 * nt)
                r = 16 * mt + 8 * half + g
                want = sum(int(values[r, j]) * powers[j] for j in range(cols)) % R
                assert total < 2**274 and (total - bias) % R == want
