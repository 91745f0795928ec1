"""Host-side native runtime: lock-free rings and sink threads, serial bus, HTTP client, convex hull, atomic file IO,
SHA-256 and the prefetching record loader (C++17, ``csrc/host/``), bound through ctypes."""
from .host import (FileSink, RecordLoader, SerialPort, SpscRing, convex_hull, gzip_inflate, http_request,  # noqa: F401
                   read_file_range, sha256, write_file_atomic)
