"""trspmm — host-side mirror of the reference's hybrid sparse operators over libtrspmm.so.

The compute lives in hand-written CUDA (csrc/, sm_100a) behind a C ABI (include/trspmm.h);
this package binds it with ctypes and uses torch only for device memory and streams.  There is
no CPU fallback: every operator raises when the library or a CUDA device is missing.
"""
from . import graphs  # noqa: F401
from ._lib import TrsError, lib_path, load  # noqa: F401
from .format import FORMAT_NAMES, Format  # noqa: F401
from .spmm import SpmmPlan, spmm_forward_host, ResidentSpmm  # noqa: F401
from .sddmm import sddmm, SddmmPlan  # noqa: F401
from .builder import build_format  # noqa: F401
from .gcn import ShardedGCN2  # noqa: F401
from . import shard  # noqa: F401
from .dataset import GCN_dataset_tcu_sptc_cuda_online, edges_to_csr, kernel_tcu_sptc_cuda_online  # noqa: F401
from .autograd import DifferentiableSpmm, transpose_csr  # noqa: F401
from . import reorder  # noqa: F401
