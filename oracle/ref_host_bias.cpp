// C-linkage access to add_rows_reference (tests/kernels/test_bias.cpp:33-45), compiled from the
// reference's source where it lies.  Test infrastructure only.
#include <tests/kernels/test_bias.cpp>

#include <cstring>

extern "C" void refhost_add_rows(std::uint16_t* out, const std::uint16_t* x, const std::uint16_t* bias, int n, int dim) {
    const std::size_t count = static_cast<std::size_t>(n) * dim;
    std::vector<__nv_bfloat16> xv(count), bv(dim);
    std::memcpy(xv.data(), x, count * 2);
    std::memcpy(bv.data(), bias, static_cast<std::size_t>(dim) * 2);
    const auto o = add_rows_reference(xv, bv, n, dim);
    std::memcpy(out, o.data(), count * 2);
}
