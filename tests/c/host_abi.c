/* The C ABI used from plain C: this file must compile as C11 against include/lfm25_b200.h, link against the library
 * and run without a GPU (it calls host-side entry points only).  Prints "ok" and exits 0, or names what failed. */
#include <stdio.h>
#include <string.h>

#include "lfm25_b200.h"

#define CHECK(condition)                                                        \
    do {                                                                        \
        if (!(condition)) {                                                     \
            printf("failed: %s (last error: %s)\n", #condition, lfm25_last_error()); \
            return 1;                                                           \
        }                                                                       \
    } while (0)

int main(void) {
    CHECK(lfm25_version() != NULL && strstr(lfm25_version(), "lfm25_b200") != NULL);
    CHECK(lfm25_splitk_workspace_elements(64) == (size_t)64 * 32 * 8 * 66);
    CHECK(lfm25_splitk_decode_splits(1, 8192, 16) == 8);
    CHECK(lfm25_bf16_own_kernel_max_rows() >= 32);

    int64_t value = -1;
    CHECK(lfm25_get_option("pdl", &value) == LFM25_OK && value == 1);
    CHECK(lfm25_set_option("no_such_switch", 1) == LFM25_ERR_INVALID_ARGUMENT);
    CHECK(strlen(lfm25_last_error()) > 0);
    CHECK(lfm25_decode_one_kernel_preferred(16, 4096, 128) == 1);

    lfm25_kv_allocator* allocator = NULL;
    lfm25_block_tables* tables = NULL;
    CHECK(lfm25_kv_allocator_create(8, 16, &allocator) == LFM25_OK);
    CHECK(lfm25_block_tables_create(2, 4, &tables) == LFM25_OK);
    CHECK(lfm25_kv_allocator_try_reserve_tokens(allocator, 40) == 3);
    uint32_t* row = lfm25_block_tables_slot(tables, 1);
    CHECK(row != NULL && row[0] == 0xffffffffu);
    CHECK(lfm25_kv_allocator_grow_sequence(allocator, 0, 33, row, 4) == 3);
    CHECK(row[0] != 0xffffffffu && row[2] != 0xffffffffu && row[3] == 0xffffffffu);
    const size_t current[2] = {33, 0};
    const size_t target[2] = {64, 48};
    CHECK(lfm25_kv_allocator_pages_short(allocator, current, target, 2) == 0);
    const size_t too_much[2] = {64, 80};
    CHECK(lfm25_kv_allocator_pages_short(allocator, current, too_much, 2) == 1);
    lfm25_kv_allocator_release_sequence(allocator, 33, row, 4);
    lfm25_kv_allocator_release_reservation(allocator, 3);
    lfm25_block_tables_destroy(tables);
    lfm25_kv_allocator_destroy(allocator);

    lfm25_dispatcher* dispatcher = NULL;
    CHECK(lfm25_dispatcher_create(4, &dispatcher) == LFM25_OK);
    const int32_t home = lfm25_dispatcher_assign_bounded(dispatcher, 1234567u, 1, 100, 250);
    CHECK(home == (int32_t)(1234567u % 4));
    CHECK(lfm25_dispatcher_load(dispatcher, (size_t)home) == 100);
    lfm25_dispatcher_mark_failed(dispatcher, (size_t)home);
    CHECK(lfm25_dispatcher_assign(dispatcher, 1234567u, 1, 10) != home);
    lfm25_dispatcher_destroy(dispatcher);

    printf("ok\n");
    return 0;
}
