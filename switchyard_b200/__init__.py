"""switchyard_b200: the mixture-of-experts layer hot path of switchyard, written from scratch
for NVIDIA B200 (sm_100a). `kernels` and `ep` mirror the reference's modules of the same
names; the kernels live in a C-ABI shared library built from `csrc/` (see `build`)."""

__all__ = ["kernels", "ep", "synthetic", "build"]
