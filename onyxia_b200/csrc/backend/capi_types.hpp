// The opaque handle types of the C ABI, shared by the translation units that implement it.
#pragma once
#include "session.hpp"

struct ox_backend {
    std::unique_ptr<oxrt::Backend> b;
};
struct ox_session {
    std::unique_ptr<oxrt::Session> s;
    std::vector<oxrt::Timing> taken;  // keeps strings alive for take_timings
};
struct ox_tensor {
    oxrt::DTensor t;
};
