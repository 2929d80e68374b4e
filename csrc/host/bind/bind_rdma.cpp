#include "bind/bind_common.h"

// Filled in by the RDMA transport translation unit when it is part of the build.
__attribute__((weak)) void bind_rdma_impl(py::module_& m);

void bind_rdma(py::module_& m)
{
    if (bind_rdma_impl) bind_rdma_impl(m);
}
