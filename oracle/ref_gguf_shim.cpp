// TEST INFRASTRUCTURE.  A thin C interface over the reference's own GGUF code (ggml/src/gguf.cpp with ggml.c), compiled
// where it lies by `make ref-gguf`: writes a model file with the reference's writer and reports where the reference's
// reader finds a tensor, so that this repository's reader (fnb_gguf_*) can be pinned against both.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "ggml.h"
#include "gguf.h"

extern "C" {

// n tensors: names[i], ggml type, n_dims[i], ne[4 i .. 4 i + 3], raw bytes data[i].  Adds a few key/value pairs of every
// kind a real model file carries (strings, an array of strings, an array of floats, scalars).  0 on success.
int ref_gguf_write(const char * path, int n, const char ** names, const int32_t * types, const int32_t * n_dims,
                   const int64_t * ne, const void ** data, uint32_t alignment) {
    gguf_context * g = gguf_init_empty();
    gguf_set_val_str(g, "general.architecture", "qwen4exp");
    gguf_set_val_u32(g, "general.alignment", alignment);
    gguf_set_val_f32(g, "qwen4exp.rope.freq_base", 1e7f);
    gguf_set_val_bool(g, "tokenizer.ggml.add_bos_token", false);
    gguf_set_val_i64(g, "some.i64", -5);
    const char * toks[4] = {"<|endoftext|>", "a", "", "bc"};
    gguf_set_arr_str(g, "tokenizer.ggml.tokens", toks, 4);
    const float scores[5] = {1.f, 2.f, 3.f, 4.f, 5.f};
    gguf_set_arr_data(g, "tokenizer.ggml.scores", GGUF_TYPE_FLOAT32, scores, 5);
    ggml_init_params ip = {ggml_tensor_overhead() * size_t(n + 1) + 4096, nullptr, true};
    ggml_context * ctx = ggml_init(ip);
    if (ctx == nullptr) return 1;
    for (int i = 0; i < n; ++i) {
        ggml_tensor * t = ggml_new_tensor(ctx, ggml_type(types[i]), n_dims[i], ne + 4 * i);
        ggml_set_name(t, names[i]);
        t->data = const_cast<void *>(data[i]);
        gguf_add_tensor(g, t);
    }
    const bool ok = gguf_write_to_file(g, path, false);
    ggml_free(ctx);
    gguf_free(g);
    return ok ? 0 : 2;
}

// Where the reference's reader finds `name`: absolute file offset of its data, ggml type, byte size.  0 on success.
int ref_gguf_find(const char * path, const char * name, int64_t * file_offset, int32_t * type, int64_t * nbytes,
                  int64_t * n_tensors) {
    gguf_init_params p = {true, nullptr};
    gguf_context * g = gguf_init_from_file(path, p);
    if (g == nullptr) return 1;
    *n_tensors = gguf_get_n_tensors(g);
    const int64_t id = gguf_find_tensor(g, name);
    int rc = 2;
    if (id >= 0) {
        *file_offset = int64_t(gguf_get_data_offset(g) + gguf_get_tensor_offset(g, id));
        *type = int32_t(gguf_get_tensor_type(g, id));
        *nbytes = int64_t(gguf_get_tensor_size(g, id));
        rc = 0;
    }
    gguf_free(g);
    return rc;
}

}  // extern "C"
