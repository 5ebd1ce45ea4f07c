/*
 * Prints the layout table of the boundary structs (sizeof / offsetof of every entry of
 * include/yvex_b200_abi_fields.h) for whichever headers it is compiled against: with
 * -DYVEX_ABI_REF and the reference's include directory, the reference's own; otherwise this
 * repository's. Identical output means a caller built against one can pass its structs to the other.
 */
#include <stddef.h>
#include <stdio.h>
#ifdef YVEX_ABI_REF
#include <yvex/backend.h>
#include <yvex/internal/backend.h>
#include <yvex/internal/moe.h>
#include <yvex/internal/quant_numeric.h>
#else
#include "yvex_b200_backend.h"
#endif

int main(void) {
#define YVEX_ABI_STRUCT(type) printf("sizeof %s %zu\n", #type, sizeof(type));
#define YVEX_ABI_FIELD(type, field) printf("offsetof %s.%s %zu\n", #type, #field, offsetof(type, field));
#include "yvex_b200_abi_fields.h"
    return 0;
}
