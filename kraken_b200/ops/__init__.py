"""Native library: build (``_build``) and ctypes binding (module ``lib``)."""
from . import lib  # noqa: F401  (the module; ``lib.lib()`` returns the loaded library)
from .lib import KrakenError, KrakenSyncTimeout, check_status, lib_path

__all__ = ["KrakenError", "KrakenSyncTimeout", "check_status", "lib", "lib_path"]
