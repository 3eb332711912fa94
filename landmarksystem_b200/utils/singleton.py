"""Metaclass that makes a class a process-wide singleton
(reference: landmark/utils/singleton.py:1-13)."""
import threading


class SingletonMeta(type):
    _instances: dict = {}
    _lock = threading.Lock()

    def __call__(cls, *args, **kwargs):
        if cls not in cls._instances:
            with cls._lock:
                if cls not in cls._instances:
                    cls._instances[cls] = super().__call__(*args, **kwargs)
        return cls._instances[cls]

    def _reset_instance(cls) -> None:
        """Forget the cached instance (used by ``destroy`` paths and tests)."""
        with cls._lock:
            cls._instances.pop(cls, None)
