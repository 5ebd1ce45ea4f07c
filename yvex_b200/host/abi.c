/*
 * Layout table of the boundary structs: one "sizeof type N" or "offsetof type.field N" line per entry
 * of include/yvex_b200_abi_fields.h. A binding (or a caller compiled against the reference's headers)
 * compares its own table with this one before it passes a struct across.
 */
#include "backend_private.h"

#include <stddef.h>
#include <stdio.h>

const char *yvex_backend_abi_layout(void) {
    static char table[16384];
    static int built;
    if (!built) {
        size_t used = 0;
#define YVEX_ABI_STRUCT(type) \
        used += (size_t)snprintf(table + used, sizeof(table) - used, "sizeof %s %zu\n", #type, sizeof(type));
#define YVEX_ABI_FIELD(type, field) \
        used += (size_t)snprintf(table + used, sizeof(table) - used, "offsetof %s.%s %zu\n", #type, #field, offsetof(type, field));
#include "yvex_b200_abi_fields.h"
#undef YVEX_ABI_STRUCT
#undef YVEX_ABI_FIELD
        built = 1;
    }
    return table;
}
