"""`import checkers_py` -- the module name the reference's callers use
(examples/FSDP_ZeRO3/train_llama3.py:11, 235-264 in the Checkers tree; the pybind module is
defined in src/python_bindings.cpp:17-35).  The three functions keep their names, argument
order and defaults; they run on libcheckers_b200.so through its C ABI.  load_and_decompress is
the reader the reference does not have."""
from checkers_b200.api import (analyze_tensors, compress_and_save, current_context, initialize_context,  # noqa: F401
                               load_and_decompress, register_tensors)

__all__ = ["initialize_context", "analyze_tensors", "compress_and_save", "load_and_decompress", "register_tensors",
           "current_context"]
