// Two builds of one kernel source. The device build (nvcc) is the product. The host build (NC_EMU, csrc/emu) compiles
// the same kernels with the host compiler and runs each CUDA thread as a fiber, for tests on machines without a GPU;
// it leaves out the launchers and replaces inline PTX by plain C++ where a kernel has any.
#pragma once
#ifdef NC_EMU
#include "../emu/cuda_emu.h"
#define NC_PDL_PROLOGUE() ((void)0)
#define NC_DYNAMIC_SHARED(type, name) type* name = static_cast<type*>(emu::dynamic_shared())
#else
// A kernel launched behind this one with programmatic serialization may start its own prologue now; the wait is a
// no-op unless this kernel was launched that way itself.
#define NC_PDL_PROLOGUE()                                           \
  do {                                                              \
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); \
    asm volatile("griddepcontrol.wait;" ::: "memory");              \
  } while (0)
#define NC_DYNAMIC_SHARED(type, name) extern __shared__ __align__(16) type name[]
#endif
