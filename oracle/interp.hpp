// TEST INFRASTRUCTURE — CPU oracle. Not part of the shipped backend: only the
// test-suite, the smoke check and the benchmark's CPU-baseline leg may link or
// call it.
//
// A C++ restatement of the reference CPU interpreter
// (crates/onyxia-ir/src/interp.rs) and of the reference backend built on it
// (crates/onyxia-backend-ref/src/lib.rs:46-107). The Rust original cannot be
// compiled where this runs, so parity is pinned against the golden vectors of
// the reference's own unit tests (interp.rs:1202-1508, decomp.rs:728-1202,
// lower_test.rs:246-305), re-expressed in tests/.
//
// Precision model (interp.rs:6-12): floats are evaluated in f64 and rounded to
// the value's dtype when each primitive stores its result; integers are
// evaluated in wrapping i64 and truncated on store.
//
// Rounding f64→f16 stands in for `half::f16::from_f64` (half 2.7.1, a Cargo
// dependency absent from the reference tree): IEEE round-to-nearest-even,
// overflow to ±inf, subnormals kept. The reference has no test that pins that
// rounding on inexact values ("parity unpinned" for that one conversion).
#pragma once
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "../onyxia_b200/csrc/ir/ir.hpp"

namespace oxref {

using ox::DType;

struct LazyDequant;

// A host tensor: dtype, shape and little-endian storage bytes
// (interp.rs:29-49). `data` may point into a module's constant pool.
struct Tensor {
    DType dtype = DType::F32;
    std::vector<size_t> shape;
    std::shared_ptr<std::vector<uint8_t>> own;
    const uint8_t* data = nullptr;
    // A Dequantize result that has not been written out yet; MatMul consumes
    // it row by row, everything else materialises it first. Values are
    // identical either way.
    std::shared_ptr<LazyDequant> lazy;

    size_t numel() const {
        size_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    size_t nbytes() const { return ox::dtype_storage_bytes(dtype, numel()); }
    static Tensor alloc(DType dt, std::vector<size_t> shape);
    static Tensor from_bytes(DType dt, std::vector<size_t> shape, const void* bytes, size_t nbytes);
    static Tensor view(DType dt, std::vector<size_t> shape, const uint8_t* bytes);
    uint8_t* mut() { return own->data(); }
};

struct LazyDequant {
    Tensor q, scales;
    bool has_zp = false;
    Tensor zp;
    size_t block_size = 0;
};

// Called for every `onyxia.AllReduce` node: sum `count` elements of dtype code `dtype` in place
// with the other tensor-parallel ranks (supplied by the test that runs the ranks).
using AllReduceHook = void (*)(void* data, uint64_t count, int32_t dtype);
AllReduceHook& allreduce_hook();

// Evaluate one primitive (interp.rs:511-799). May bind late symbols.
Tensor eval_prim(const ox::Prim& p, const std::vector<const Tensor*>& ins, ox::Bindings& bindings);
// Write out a lazily dequantised tensor.
void materialize(Tensor& t);

// Evaluate a pure-primitive module (interp.rs:419-495).
std::vector<std::pair<std::string, Tensor>> eval(const ox::Module& m,
                                                 const std::vector<std::pair<std::string, Tensor>>& inputs);

// ≙ RefBackend::prepare / RefSession::run (onyxia-backend-ref/src/lib.rs:46-85).
struct RefSession {
    ox::Module module;  // fully inlined, validated
    std::vector<ox::NodeId> order;
    std::vector<std::vector<ox::ValueId>> deaths;
    std::vector<std::pair<std::string, Tensor>> run(const std::vector<std::pair<std::string, Tensor>>& inputs) const;
};
RefSession prepare(ox::Module m);

// Number of OpenMP threads used for the big loops (1 = the reference's
// single-threaded behaviour; per-output accumulation order never changes).
void set_threads(int n);
int get_threads();

}  // namespace oxref
