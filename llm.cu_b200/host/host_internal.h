// Declarations shared by the host-side translation units (not part of the public surface).
#pragma once

#include <functional>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/llama3.h"

namespace llmb {

// Calls fn(tensor, layer, slot) for every tensor of the model: layer = -1 and slot =
// LLMB_SID_EMBED / LLMB_SID_LM_HEAD / LLMB_SID_NORM for the three global tensors, else the layer
// index and the LLMB_SLOT_* of the tensor.  Order: the reference's _m_component_tensor_operation
// (src/llama3/llama3.cu:257-277).
void for_each_tensor(Llama3 *m, const std::function<void(Tensor *, int, int)> &fn);

// Where a tensor's payload lies in a checkpoint shard: recorded by the loader, read by to_cuda.
struct TensorSource {
    int file = -1;                 // index into ModelPriv::files
    unsigned long long offset = 0; // absolute byte offset of element 0
};

// Host-side state behind Llama3::priv.
struct ModelPriv {
    std::vector<std::string> files;
    std::unordered_map<const Tensor *, TensorSource> sources;
    bool streaming = true;   // payloads stay in the files until to_cuda reads this rank's windows
    // figures of the last to_cuda()
    double upload_seconds = 0.0;
    unsigned long long bytes_read = 0, bytes_uploaded = 0, staging_bytes = 0;
};

ModelPriv *model_priv(Llama3 *m);  // created on first use; freed by free_llama3

}  // namespace llmb
