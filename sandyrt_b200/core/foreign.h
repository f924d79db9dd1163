// Parts and architectures implemented outside this library, behind the C interface's callbacks.
#pragma once

#include <string>

#include "c_api.h"
#include "parts.h"

namespace sandy {

void register_foreign_part(const std::string& family, const std::string& kind, const SandyForeignPart& vtable, void* user);
void register_foreign_architecture(const std::string& name, sandy_json_fn parse, sandy_json_fn describe, void* user);

// The error a callback reported with sandy_set_callback_error (cleared by reading).
void set_callback_error(const std::string& kind, const std::string& message);
[[noreturn]] void throw_callback_error(const std::string& where);

// A step as the callbacks see it.  The arrays it points at live as long as the object.
struct StepViewHolder {
    explicit StepViewHolder(StepContext& ctx);
    SandyStepView view;
    std::vector<const int*> tables;
};

}  // namespace sandy
