"""Process-level helpers (reference: landmark/nerf_components/utils/system_utils.py:17-45)."""
import os
import sys
from datetime import datetime


def mkdir_p(path):
    os.makedirs(path, exist_ok=True)


def searchForMaxIteration(folder):
    return max(int(name.split("_")[-1]) for name in os.listdir(folder))


class _StampedStream:
    def __init__(self, stream):
        self._stream = stream
        self._at_line_start = True

    def write(self, text):
        for piece in text.splitlines(keepends=True):
            if self._at_line_start and piece.strip():
                self._stream.write(datetime.now().strftime("[%d/%m %H:%M:%S] "))
            self._stream.write(piece)
            self._at_line_start = piece.endswith("\n")

    def flush(self):
        self._stream.flush()

    def __getattr__(self, name):
        return getattr(self._stream, name)


def set_print_with_timestamp():
    """Prefix every stdout line with a timestamp (idempotent)."""
    if not isinstance(sys.stdout, _StampedStream):
        sys.stdout = _StampedStream(sys.stdout)
