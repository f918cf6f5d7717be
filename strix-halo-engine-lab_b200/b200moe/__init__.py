"""Host-side Python binding of the B200 MoE FFN library (ctypes over the C ABI of include/b200moe.h)."""
