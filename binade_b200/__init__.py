"""binade_b200: Binade's lossless BF16 weight compression, hot path on NVIDIA B200 (sm_100a).

Same Python surface as the reference package for the path it covers: `bf16`, `format`, `rice`,
`st`, `pack`, `unpack` on the host side (tensor-level round trip: `pack.pack(w)` and
`unpack.unpack(p)`); `binade_b200.cuda.r4` (transcode, R4Linear, convert) and
`binade_b200.cuda.moe` (R4SwitchGLU) at run time. Host code calls hand-written CUDA through the
C ABI declared in include/binade_b200.h; there is no CPU fallback for anything that runs on the
GPU in the reference's fast path.
"""

__version__ = "0.1.0"

