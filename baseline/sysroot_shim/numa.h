/* Stand-in for the libnuma development header, which this image does not ship.
 * The reference includes <numa.h> from a common header, but with BUILD_RDMA=OFF
 * none of its NUMA calls are compiled, so an empty header is enough to build the
 * unmodified NVLink endpoint for the comparison arm of bench.py. */
#pragma once
