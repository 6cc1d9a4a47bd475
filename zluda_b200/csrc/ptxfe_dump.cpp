// Host translation unit of the library: the canonical dump (ptx_dump.h) compiled by the host compiler.
#define PTX_HD
#define PTX_TABLE static const
#include "ptx_dump.h"

std::string ptxfe_dump_module_impl(const PtxBatchView& v, uint32_t m, int* status) { return ptxdump::dump_module(v, m, status); }
uint64_t ptxfe_dump_hash_impl(const PtxBatchView& v, uint32_t m, int* status) {
    uint64_t h = 0;
    ptxdump::dump_module(v, m, status, &h);
    return h;
}
