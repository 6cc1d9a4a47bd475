// Host translation unit of the library: the canonical dump (ptx_dump.h) compiled by the host compiler.
#define PTX_HD
#define PTX_TABLE static const
#include "ptx_ast.h"

std::string ptxfe_dump_module_impl(const PtxBatchView& v, uint32_t m, int* status) { return ptxdump::dump_module(v, m, status); }
// the dump by way of the tree: records -> ptxast::Module -> text
std::string ptxfe_dump_module_tree_impl(const PtxBatchView& v, uint32_t m, int* status) {
    ptxast::Module mod;
    ptxast::materialize(v, m, &mod);
    if (status) *status = mod.have_module ? 0 : 1;
    return ptxast::print(v, m, mod);
}
// builds and drops the tree of module m; returns the number of nodes built
uint64_t ptxfe_materialize_impl(const PtxBatchView& v, uint32_t m) {
    ptxast::Module mod;
    ptxast::materialize(v, m, &mod);
    return mod.nodes + mod.directives.size();
}
uint64_t ptxfe_dump_hash_impl(const PtxBatchView& v, uint32_t m, int* status) {
    uint64_t h = 0;
    ptxdump::dump_module(v, m, status, &h);
    return h;
}
