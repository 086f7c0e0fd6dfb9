"""recstore_b200: a Blackwell-native (sm_100a) embedding parameter server and
recommendation / knowledge-graph training framework with the capabilities of RecStore.

Sub-packages
------------
``ops``       native kernels (tcgen05 GEMM, fused embedding forward/backward, interaction, losses)
``parallel``  in-box NVLink transport: peer windows, flags, all-reduce, sharding policies
``models``    DLRM (dot / DCNv2), SimpleDLRM, knowledge-graph embedding models
``utils``     synthetic data, timers, logging, liveness (heartbeat), profiler windows
``cache``     cached embeddings, GPU cache, tiered and lookahead tables
``ps``        parameter server: shard process, clients (TCP, gRPC, NVLink), load generation
``cli``       drivers (DLRM, KG training / inference / distributed, micro-benchmarks)
``baseline``  PyTorch + NCCL restatements of the reference algorithms (oracle and measured baseline)

The native library is built in-tree (``python -m recstore_b200.build``) and bound with ctypes.
"""
__version__ = "0.2.0"

from . import _lib  # noqa: F401
from ._lib import RecStoreError, DeviceStatusError  # noqa: F401

from .kvstore import kvinit, get_kvstore, AbsKVStore, ShmKVStore  # noqa: F401,E402
from .dist_tensor import DistTensor, DistEmbedding, HbmDistEmbedding, PartitionPolicy  # noqa: F401,E402
from . import dist_opt as DistOpt  # noqa: F401,E402
from .dist_opt import SparseSGD, SparseAdagrad, SparseRowWiseAdaGrad  # noqa: F401,E402
from .ipc import IPCTensorFactory, SlicedTensor, MultiProcessBarrierFactory, Mfence  # noqa: F401,E402
from .utils.liveness import Heartbeat, RankLostError  # noqa: F401,E402
