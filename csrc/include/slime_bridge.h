/* A C function table over the host runtime's endpoints, for native code that cannot include the C++ headers of the
 * runtime or link against its Python module: the torch.distributed backend (csrc/torch/slime_backend.cpp) is built
 * against libtorch with torch's own compiler settings and reaches the endpoints only through this table. The Python
 * module hands out the table's address (`_slime_c.bridge_table()`); every pointer in it stays valid while the module is
 * loaded. Strings returned by the table are released with `free_string`. Status codes are those of the futures:
 * 0 ok, 402 timed out, 403 failed. */
#ifndef SLIME_BRIDGE_H
#define SLIME_BRIDGE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLIME_BRIDGE_VERSION 1

typedef struct SlimeBridge {
    int version;
    /* transport: "tcp", "rdma" or "" (RDMA when a verbs provider with a device exists, else TCP). `rank` picks the NIC
     * round robin. Returns NULL and fills err (if given) on failure. */
    void* (*endpoint_create)(const char* transport, const char* bind_host, int rank, char* err, size_t err_len);
    void (*endpoint_destroy)(void* ep); /* shuts the endpoint down first */
    char* (*endpoint_info)(void* ep);   /* JSON text */
    int (*endpoint_connect)(void* ep, const char* info_json, char* err, size_t err_len);
    const char* (*endpoint_kind)(void* ep);
    void* (*send)(void* ep, uintptr_t ptr, size_t length); /* -> future */
    void* (*recv)(void* ep, uintptr_t ptr, size_t length); /* -> future */
    int (*future_wait)(void* future, int64_t timeout_ms);
    int (*future_done)(void* future);
    void (*future_free)(void* future);
    void (*free_string)(char* s);
} SlimeBridge;

#ifdef __cplusplus
}
#endif
#endif
