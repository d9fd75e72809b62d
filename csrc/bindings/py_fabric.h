// The Python-side owner of a transfer engine, shared by the binding translation units that take
// an engine as an argument.
#pragma once

#include <memory>

#include "../core/error.h"
#include "../fabric/transfer_engine.h"

struct PyEngine {
  std::unique_ptr<pplx::fabric::TransferEngine> engine;
  pplx::fabric::TransferEngine& get() {
    if (!engine) throw pplx::Error(pplx::ErrorKind::kWorkerDown, "the transfer engine was stopped");
    return *engine;
  }
};
