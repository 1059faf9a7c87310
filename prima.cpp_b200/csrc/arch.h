// prima.cpp_b200/csrc/arch.h — the table of model architectures this library runs.  Two families:
//   ARCH_KQUANT   one fixed transformer graph over k-quant GGUF weights (engine.cu): "llama", "qwen2"
//   ARCH_LAYERS   the configuration lists the layers, each with a sequence mixer and an optional feed-forward, over dense
//                 f32 / bf16 weights from a safetensors file (layers.cu): "Vamidra", "Mumizen", "Sapudra", "Zevedra"
// A loader looks the architecture string of its container up here (GGUF: general.architecture; configuration file: "architecture")
// and takes the family's path; an unknown string is PB200_ENOTSUP.
#pragma once
#include <string>

namespace pb {

struct Json;
struct LayerList;

enum : int { ARCH_KQUANT = 0, ARCH_LAYERS = 1 };

struct ArchEntry {
    const char * name;
    int family;
    // ARCH_KQUANT
    int rope_mode;   // 0 = NORM, 2 = NEOX
    // ARCH_LAYERS: reads the configuration into the layer list (sizes, constants, order of layer runs); returns 0 or a PB200_E* code
    int (*configure)(const Json & cfg, LayerList & ll, std::string & err);
    // ARCH_LAYERS: maps a tensor name of the checkpoint to its place in the model; returns false for a name the design does not have
    bool (*resolve)(LayerList & ll, const std::string & name, struct TensorPlace & out);
};

const ArchEntry * arch_find(const char * name);
int arch_count();
const ArchEntry * arch_at(int i);

}  // namespace pb
