/* TEST INFRASTRUCTURE ONLY.  Stand-in for the bounds-checked C library header the reference's host code includes
 * (it is not part of the reference tree and not installed here): the two calls it uses, with their documented
 * contract -- return 0 on success, non-zero when an argument is invalid or the destination is too small. */
#ifndef RECSDK_ORACLE_SECUREC_SHIM_H
#define RECSDK_ORACLE_SECUREC_SHIM_H
#include <stddef.h>
#include <string.h>
typedef int errno_t;
#ifndef EOK
#define EOK 0
#endif
static inline errno_t memcpy_s(void* dest, size_t dest_max, const void* src, size_t count)
{
    if (dest == NULL || src == NULL || count > dest_max) return 1;
    memcpy(dest, src, count);
    return 0;
}
static inline errno_t memset_s(void* dest, size_t dest_max, int c, size_t count)
{
    if (dest == NULL || count > dest_max) return 1;
    memset(dest, c, count);
    return 0;
}
#endif
