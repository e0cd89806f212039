"""C++ host side of the fast path (tcbnn_host.hpp: the reference's layer classes on the C ABI)
and the generic driver built on it (fast_runner.cpp)."""
