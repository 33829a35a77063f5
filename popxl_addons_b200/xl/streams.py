"""`xl.streams` (popxl/streams.py): host-to-device and device-to-host streams."""
from .buffers import DeviceToHostStream, HostToDeviceStream, _Stream as Stream, d2h_stream, h2d_stream  # noqa: F401

__all__ = ["Stream", "HostToDeviceStream", "DeviceToHostStream", "h2d_stream", "d2h_stream"]
