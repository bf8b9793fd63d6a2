// Device side of a reference-named extension module: the FP32 kernels of the library are
// compiled straight into the module, so the two-file build the reference's scripts perform
// (load(sources=[<wrapper>.cpp, <kernel>.cu]), naive/test.py:5-11) yields a working module
// with no extra link flags.
#pragma once
#include "../csrc/sgemm_f32.cu"
#include "../csrc/status.cu"
