from .control import (get_comm_stream, get_local_world_pg, get_local_world_size)
from .heap import CudaHeap, HostShmHeap, SymmetricHeap, create_heap
from .registry import SymmBufferRegistry
from .status import Heartbeat, OdcBoundsError, OdcError, OdcTimeoutError, PeerFailure
from .transport import HostShmTransport, InterNodeTransport, NvlinkP2PTransport, Transport, make_transport
