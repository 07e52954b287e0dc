"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Real EXL3 checkpoints are not available offline, so every tensor is drawn from a numpy Generator:
  - trellis codes: uniform random bytes (any bit pattern is a valid tile of the format);
  - suh (input side): +-1 as FP16, sign uniform;  svh (output side): +-U(0.005, 0.03) as FP16, sign uniform;
  - tokens: bfloat16 of N(0, 1);  router scores: FP32 N(0, 1);  reduction partials: FP32 N(0, 0.05^2);
  - per-expert stored width from {2, 3, 4} with probabilities {0.2, 0.5, 0.3}.
The same arrays feed the CUDA path and the CPU oracle.
"""
import numpy as np


def bits_x2(stored_width):
    if 1 <= stored_width <= 8:
        return 2 * stored_width
    if stored_width % 16 == 8 and stored_width < 128:
        return stored_width // 8
    return 0


def code_bytes(inputs, outputs, stored_width):
    return inputs * outputs // 16 * bits_x2(stored_width)


def matrix_bytes(inputs, outputs, stored_width):
    return code_bytes(inputs, outputs, stored_width) + 2 * (inputs + outputs)


def exl3_matrix(rng, inputs, outputs, stored_width):
    """The stored bytes of one matrix: codes, suh[inputs], svh[outputs]."""
    codes = rng.integers(0, 256, size=code_bytes(inputs, outputs, stored_width), dtype=np.uint8)
    suh = np.where(rng.integers(0, 2, size=inputs) == 0, 1.0, -1.0).astype(np.float16)
    svh = (rng.uniform(0.005, 0.03, size=outputs) * np.where(rng.integers(0, 2, size=outputs) == 0, 1.0, -1.0))
    return np.concatenate([codes, suh.view(np.uint8), svh.astype(np.float16).view(np.uint8)])


def slice_matrix(matrix, inputs, outputs, stored_width, in_begin, in_count, out_begin, out_count):
    """Lossless slice of a stored matrix in numpy (rows of 16 inputs, tiles of 16 outputs; all multiples of 128)."""
    tile = 16 * bits_x2(stored_width)
    codes = matrix[:code_bytes(inputs, outputs, stored_width)].reshape(inputs // 16, outputs // 16, tile)
    kept = codes[in_begin // 16:(in_begin + in_count) // 16, out_begin // 16:(out_begin + out_count) // 16]
    scales = matrix[code_bytes(inputs, outputs, stored_width):]
    return np.concatenate([kept.reshape(-1), scales[2 * in_begin:2 * (in_begin + in_count)],
                           scales[2 * (inputs + out_begin):2 * (inputs + out_begin + out_count)]])


def to_bfloat16(values):
    """float32 -> bfloat16 bits (uint16), to nearest even."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def from_bfloat16(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def tokens(rng, rows, hidden):
    return to_bfloat16(rng.normal(0.0, 1.0, size=(rows, hidden)).astype(np.float32))


def expert_widths(rng, expert_count, choices=(2, 3, 4), probabilities=(0.2, 0.5, 0.3)):
    return rng.choice(np.array(choices, dtype=np.uint32), size=expert_count, p=probabilities).astype(np.uint32)


def zipf_scores(rng, rows, expert_count, exponent=1.1):
    """Router scores whose top picks follow a Zipf(exponent) expert popularity (Gumbel top-k of log popularity)."""
    popularity = -exponent * np.log(np.arange(1, expert_count + 1, dtype=np.float64))
    gumbel = rng.gumbel(size=(rows, expert_count))
    return (popularity[None, :] + gumbel).astype(np.float32)


def mx_matrix(rng, outputs, inputs):
    """Stored bytes of one WEIGHT_FORMAT_E2M1_SCALED matrix of the original-weights profile: uniform E2M1 nibbles
    (every byte pattern is a valid pair of codes), then E8M0 scale codes 127 + e with e uniform in [-8, -4], one per
    32 inputs. Independent draws, so the stored order of the format needs no permutation here."""
    words = rng.integers(0, 256, size=outputs * inputs // 2, dtype=np.uint8)
    scales = (127 + rng.integers(-8, -3, size=outputs * inputs // 32)).astype(np.uint8)
    return np.concatenate([words, scales])


def e4m3_matrix(rng, outputs, inputs):
    """Stored bytes of one WEIGHT_FORMAT_E4M3_SCALED matrix: E4M3 bytes that are numbers (0x7F and 0xFF never occur),
    then one E8M0 scale code per 32 outputs by 32 inputs, 127 + e with e uniform in [-9, -5] (weights of about the
    size of the profile's routed experts'). Independent draws, so the format's stored order needs no permutation."""
    codes = rng.integers(0, 127, size=outputs * inputs, dtype=np.uint8)
    codes |= (rng.integers(0, 2, size=outputs * inputs, dtype=np.uint8) << 7)
    scales = (127 + rng.integers(-9, -4, size=(outputs + 31) // 32 * (inputs // 32))).astype(np.uint8)
    return np.concatenate([codes, scales])


def e4m3_block128_matrix(rng, outputs, inputs):
    """Stored bytes of one WEIGHT_FORMAT_E4M3_BLOCK128 matrix (the block-scaled FP8 of the original-weights profile):
    E4M3 bytes that are numbers, then one FP32 scale per 128 outputs by 128 inputs drawn U(0.5, 2) / 448."""
    codes = rng.integers(0, 127, size=outputs * inputs, dtype=np.uint8)
    codes |= (rng.integers(0, 2, size=outputs * inputs, dtype=np.uint8) << 7)
    scales = (rng.uniform(0.5, 2.0, size=(outputs + 127) // 128 * (inputs // 128)) / 448.0).astype(np.float32)
    return np.concatenate([codes, scales.view(np.uint8)])
