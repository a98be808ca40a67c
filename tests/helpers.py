"""Shared helpers of the GPU parity tests: seeded inputs, byte-level comparisons, the
python restatement of the GEMM scale-factor layout."""
import numpy as np
import torch


def seeded_bf16(shape, seed, std=1.0):
    """Seeded N(0, std) tensor generated on the CPU in fp32 and rounded to bf16, so the oracle
    and the kernel see identical bytes. Returns (torch bf16 CPU tensor, float32 numpy view)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    t = (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
    return t, t.float().numpy()


def from_bits(u16: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).view(torch.bfloat16)


def np_u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().view(torch.uint8).numpy()


def padded_chunks(k_blocks: int) -> int:
    return ((k_blocks + 3) // 4 + 3) // 4 * 4


def swizzle_scales_ref(s: np.ndarray, rows: int) -> np.ndarray:
    """Row-major scale bytes [>=rows, KB] -> the 128x4-chunk layout, zero padded."""
    kb = s.shape[1]
    rb, kc = (rows + 127) // 128, padded_chunks(kb)
    full = np.zeros((rb * 128, kc * 4), dtype=np.uint8)
    full[:rows, :kb] = s[:rows]
    # [rb, 4(r/32), 32(r%32), kc, 4] -> [rb, kc, 32, 4, 4]
    v = full.reshape(rb, 4, 32, kc, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(v).reshape(-1)


def mismatch(a: np.ndarray, b: np.ndarray) -> int:
    assert a.shape == b.shape, (a.shape, b.shape)
    return int((a != b).sum())


def unswizzle_scales_ref(swz: np.ndarray, rows: int, k_blocks: int) -> np.ndarray:
    """Inverse of swizzle_scales_ref restricted to the valid [rows, k_blocks] region."""
    rb, kc = (rows + 127) // 128, padded_chunks(k_blocks)
    v = swz.reshape(rb, kc, 32, 4, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(v).reshape(rb * 128, kc * 4)[:rows, :k_blocks]
