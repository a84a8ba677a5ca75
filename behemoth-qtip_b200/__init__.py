"""qtip_b200: B200 (sm_100a) implementation of the QTIP 2-bit trellis codec hot path behind a C ABI.

`codec` mirrors the quantizer-side kernel interface (k_viterbi_fwd, k_ldlq_prep, ldlq_gpu, ...), `linear` the
runtime's QTIP linear operator (QtipMatrix, qtip_prepare / qtip_multiply / qtip_finish / qtip_forward, ...).
PyTorch is used only for device memory, streams and torch.distributed.
"""
from ._lib import (LIB_PATH, Library, QtipCheckpointLinear, QtipError, QtipGroupLinear, QtipMatrix,  # noqa: F401
                   QtipTpExchange, exported_names, lib)
from . import checkpoint, codec, linear, sharding, synth, tp  # noqa: F401
