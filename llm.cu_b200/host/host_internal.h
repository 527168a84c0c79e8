// Declarations shared by the host-side translation units (not part of the public surface).
#pragma once

#include <functional>

#include "../../include/llama3.h"

namespace llmb {

// Calls fn(tensor, layer, slot) for every tensor of the model: layer = -1 and slot =
// LLMB_SID_EMBED / LLMB_SID_LM_HEAD / LLMB_SID_NORM for the three global tensors, else the layer
// index and the LLMB_SLOT_* of the tensor.  Order: the reference's _m_component_tensor_operation
// (src/llama3/llama3.cu:257-277).
void for_each_tensor(Llama3 *m, const std::function<void(Tensor *, int, int)> &fn);

}  // namespace llmb
