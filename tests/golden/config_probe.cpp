// Driver for the reference's own configuration parser (src/model/config.cpp of
// RicardoMin/Qwen3-Runtime-ByYourself), compiled on the CPU by make_config_golden.py.
// For every file named on the command line it prints one line:
//   OK <layers> <hidden> <q_size> <kv_size> <group> <tied> <theta> <eps>     or     ERR <message>
#include <exception>
#include <iostream>

#include "qwen3/model/config.h"

int main(int argc, char** argv) {
    for (int i = 1; i < argc; ++i) {
        try {
            const auto c = qwen3::load_model_config(argv[i]);
            std::cout << "OK " << c.num_hidden_layers << " " << c.hidden_size << " " << c.q_projection_size() << " "
                      << c.kv_projection_size() << " " << c.query_heads_per_kv_head() << " "
                      << (c.tie_word_embeddings ? 1 : 0) << " " << c.rope_theta << " " << c.rms_norm_eps << "\n";
        } catch (const std::exception& e) {
            std::cout << "ERR " << e.what() << "\n";
        }
    }
    return 0;
}
