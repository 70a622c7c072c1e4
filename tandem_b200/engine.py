"""Loader of the native host runtime (tandem_b200._host), built in-tree on first
use.  Same role as the reference's tandem/engine.py:22-37: `lib()` returns the
module that exposes SharedMemory, Channel, Engine, Work, _move_check, Timeout and
NotImplemented."""

import functools
import importlib
import os


@functools.cache
def lib():
    from .utils import build

    build.build_host(verbose=os.environ.get("TANDEM_BUILD_VERBOSE") == "1")
    return importlib.import_module("tandem_b200._host")
