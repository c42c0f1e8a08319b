// Definitions of the opaque C handles, shared by every translation unit that
// exports C symbols (capi/src/handles.rs:6-44 in the reference).
#pragma once
#include "ta_core.hpp"

using namespace ta;

struct ta_context {
  std::shared_ptr<Context> ctx;
};
struct ta_executor {
  std::shared_ptr<Context> ctx;
  std::unique_ptr<Executor> exec;
};
struct ta_tensor {
  Tensor tensor;
};
struct ta_prepared {
  std::unique_ptr<PreparedOps> prepared;
  std::shared_ptr<Context> ctx;
};
struct ta_pos_cell {
  PosCell cell;
};
struct ta_token_ids {
  TokenIds ids;
};
struct ta_comm {
  std::unique_ptr<Comm> comm;
};


// Thread-local error string of the C ABI (capi/src/error.rs:8-32).
void ta_set_last_error(const char *msg);
