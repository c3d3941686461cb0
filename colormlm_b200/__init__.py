"""B200 (sm_100a) implementation of the S14 MoE expert hot path behind the reference's
operator / page-pool interface.  ``colormlm_b200.s14`` is the Python mirror of that
interface over the C ABI in ``include/polaris_s14_cuda.h``; ``pages`` describes the
in-slot page layout; ``synth`` makes seeded synthetic inputs.  Importing the package
loads ``libpolaris_s14_cuda.so`` lazily and fails loudly if it has not been built."""
from . import _lib, pages, synth  # noqa: F401
from ._lib import (ACCUM_PAIRWISE, ACCUM_REFERENCE, EXPERT_PAGE_BYTES, PAGE_FP8, PAGE_MXFP4,  # noqa: F401
                   SCALE_F32, SCALE_UE8M0, SCORE_SIGMOID, SCORE_SQRT_SOFTPLUS,
                   SHARED_EXPERT_PAGE_BYTES, S14Error)

__version__ = "0.1.0"
