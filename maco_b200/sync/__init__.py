"""Stream management and signal/wait synchronisation (reference: maco/sync/__init__.py:7-30)."""
from .signal_wait import DeviceSignal, OverlapContext, Signal, SignalWait, create_signal
from .stream_manager import StreamManager, get_comm_stream, get_compute_stream

__all__ = ["StreamManager", "get_compute_stream", "get_comm_stream", "Signal", "SignalWait", "create_signal",
           "OverlapContext", "DeviceSignal"]
