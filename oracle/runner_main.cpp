// Entry point for the reference's kernel test sources when they are compiled
// with stub_runner/gtest/gtest.h and linked against a replacement library.
#include <gtest/gtest.h>

int main() { return ::rh_gtest_runner::run_all(); }
