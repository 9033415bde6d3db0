// Shared between the libraries that implement parts of onyxia_cuda.h: the
// opaque module handle and the error plumbing of the C boundary.
#pragma once
#include <string>

#include "../../../include/onyxia_cuda.h"
#include "ir.hpp"

// The opaque handle of the C ABI: a module under construction.
struct ox_module {
    ox::GraphBuilder b;
};

namespace ox {
extern thread_local std::string g_last_error;
int set_error(const Error& e);
int set_error(ErrKind k, const std::string& msg);
DimExpr dim_from_c(const ox_dimexpr& e);
Prim prim_from_c(const ox_prim_desc& d);
}  // namespace ox
