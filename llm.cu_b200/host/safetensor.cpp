// Safetensors shard reader: the reference's src/safetensor/safetensor.cu re-implemented.
//
//   load_safetensor_weights   safetensor.cu:16-31   open, read header, load every tensor entry
//   header                    safetensor.cu:33-50   u64 little-endian length + JSON text
//   entry -> struct slot      safetensor.cu:82-162  substring match on the key, layer number =
//                                                   third dot-separated field, payload at
//                                                   8 + header_size + data_offsets[0]
//
// The reference parses the header with the vendored cJSON; this file has its own small parser
// for the subset safetensors headers use (one object of objects with "dtype", "shape",
// "data_offsets"; anything else, e.g. "__metadata__", is skipped).  Unlike the reference it
// checks dtype (BF16 is converted at upload, F16 passes through, anything else is an error),
// payload size against shape, offsets against the file size, and the layer index.
//
// By default the loader only records where each payload lies (file, offset): to_cuda then reads
// this rank's window of every tensor straight from the file into pinned staging buffers, so the host
// never holds more than those buffers.  With llama3_set_streaming(m, 0) the payload is read here
// into Tensor::bf16_tensor, as the reference does (safetensor.cu:140-155), and kept until to_cuda.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/llama3.h"
#include "host_internal.h"

namespace llmb {
void set_last_error(const char *msg);
}

namespace {

struct Entry {
    std::string name, dtype;
    std::vector<long long> shape;
    unsigned long long begin = 0, end = 0;
    bool has_dtype = false, has_shape = false, has_offsets = false;
};

class HeaderParser {
  public:
    HeaderParser(const char *s, size_t n) : p_(s), end_(s + n) {}

    bool parse(std::vector<Entry> &out) {
        ws();
        if (!eat('{')) return false;
        ws();
        if (peek() == '}') { ++p_; return true; }
        for (;;) {
            Entry e;
            ws();
            if (!string(e.name)) return false;
            ws();
            if (!eat(':')) return false;
            ws();
            if (peek() == '{') {
                if (!entry(e)) return false;
                if (e.has_dtype && e.has_shape && e.has_offsets) out.push_back(e);  // safetensor.cu:70
            } else if (!skip_value()) {
                return false;
            }
            ws();
            if (eat(',')) continue;
            return eat('}');
        }
    }

  private:
    const char *p_, *end_;
    char peek() const { return p_ < end_ ? *p_ : '\0'; }
    bool eat(char c) {
        if (p_ < end_ && *p_ == c) { ++p_; return true; }
        return false;
    }
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    bool string(std::string &out) {
        if (!eat('"')) return false;
        out.clear();
        while (p_ < end_ && *p_ != '"') {
            if (*p_ == '\\') {
                if (++p_ >= end_) return false;
                switch (*p_) {
                    case 'n': out.push_back('\n'); break;
                    case 't': out.push_back('\t'); break;
                    case 'u':  // keep the escape verbatim; tensor names never need it
                        out.append("\\u");
                        break;
                    default: out.push_back(*p_);
                }
                ++p_;
            } else {
                out.push_back(*p_++);
            }
        }
        return eat('"');
    }
    bool number(double &v) {
        const char *s = p_;
        while (p_ < end_ && (strchr("+-.eE", *p_) || (*p_ >= '0' && *p_ <= '9'))) ++p_;
        if (p_ == s) return false;
        v = strtod(std::string(s, p_).c_str(), nullptr);
        return true;
    }
    bool int_array(std::vector<long long> &out) {
        if (!eat('[')) return false;
        ws();
        if (eat(']')) return true;
        for (;;) {
            double v;
            ws();
            if (!number(v)) return false;
            out.push_back((long long)v);
            ws();
            if (eat(',')) continue;
            return eat(']');
        }
    }
    bool skip_value() {
        ws();
        char c = peek();
        if (c == '"') { std::string s; return string(s); }
        if (c == '{' || c == '[') {
            char close = c == '{' ? '}' : ']';
            ++p_;
            ws();
            if (eat(close)) return true;
            for (;;) {
                ws();
                if (c == '{') {
                    std::string k;
                    if (!string(k)) return false;
                    ws();
                    if (!eat(':')) return false;
                }
                if (!skip_value()) return false;
                ws();
                if (eat(',')) continue;
                return eat(close);
            }
        }
        if (!strncmp(p_, "true", 4) && end_ - p_ >= 4) { p_ += 4; return true; }
        if (!strncmp(p_, "false", 5) && end_ - p_ >= 5) { p_ += 5; return true; }
        if (!strncmp(p_, "null", 4) && end_ - p_ >= 4) { p_ += 4; return true; }
        double v;
        return number(v);
    }
    bool entry(Entry &e) {
        if (!eat('{')) return false;
        ws();
        if (eat('}')) return true;
        for (;;) {
            std::string key;
            ws();
            if (!string(key)) return false;
            ws();
            if (!eat(':')) return false;
            ws();
            if (key == "dtype" && peek() == '"') {
                if (!string(e.dtype)) return false;
                e.has_dtype = true;
            } else if (key == "shape" && peek() == '[') {
                if (!int_array(e.shape)) return false;
                e.has_shape = true;
            } else if (key == "data_offsets" && peek() == '[') {
                std::vector<long long> off;
                if (!int_array(off) || off.size() != 2 || off[0] < 0 || off[1] < off[0]) return false;
                e.begin = (unsigned long long)off[0];
                e.end = (unsigned long long)off[1];
                e.has_offsets = true;
            } else if (!skip_value()) {
                return false;
            }
            ws();
            if (eat(',')) continue;
            return eat('}');
        }
    }
};

int fail(int code, const char *fmt, const char *a = "", const char *b = "") {
    char msg[512];
    snprintf(msg, sizeof msg, fmt, a, b);
    llmb::set_last_error(msg);
    return code;
}

// safetensor.cu:164-191: the layer number is the third dot-separated field of the key.
int layer_of_key(const std::string &key) {
    size_t a = key.find('.');
    if (a == std::string::npos) return -1;
    size_t b = key.find('.', a + 1);
    if (b == std::string::npos) return -1;
    size_t c = key.find('.', b + 1);
    std::string field = key.substr(b + 1, c == std::string::npos ? std::string::npos : c - b - 1);
    if (field.empty() || field.find_first_not_of("0123456789") != std::string::npos) return -1;
    return atoi(field.c_str());
}

// safetensor.cu:99-123: which struct slot a key names.  Same substrings, same precedence.
Tensor *slot_of_key(Llama3 *m, const std::string &key, int *needs_layer) {
    static const char *layer_keys[] = {"input_layernorm", "down_proj", "gate_proj", "up_proj", "post_attention_layernorm",
                                       "k_proj", "o_proj", "q_proj", "v_proj"};
    *needs_layer = 0;
    for (int i = 0; i < 9; ++i) {
        if (key.find(layer_keys[i]) == std::string::npos) continue;
        *needs_layer = 1;
        int layer = layer_of_key(key);
        if (layer < 0 || layer >= m->n_layers) return nullptr;
        Llama3Layer *l = m->layers[layer];
        switch (i) {
            case 0: return l->input_layernorm;
            case 1: return l->mlp_down_proj;
            case 2: return l->mlp_gate_proj;
            case 3: return l->mlp_up_proj;
            case 4: return l->post_attention_layernorm;
            case 5: return l->self_attn_k_proj;
            case 6: return l->self_attn_o_proj;
            case 7: return l->self_attn_q_proj;
            default: return l->self_attn_v_proj;
        }
    }
    if (key.find("embed_tokens") != std::string::npos) return m->embed_tokens;
    if (key.find("model.norm") != std::string::npos) return m->norm;
    if (key.find("lm_head") != std::string::npos) return m->lm_head;
    return nullptr;
}

}  // namespace

extern "C" int llama3_load_safetensors(Llama3 *m, const char *filename) {
    if (!m || !filename) return fail(LLMB_ERR_INVALID, "load_safetensor_weights: null argument");
    FILE *fp = fopen(filename, "rb");
    if (!fp) return fail(LLMB_ERR_IO, "Error: An Error Occurred while opening %s", filename);
    struct Closer {
        FILE *f;
        ~Closer() { fclose(f); }
    } closer{fp};

    fseek(fp, 0, SEEK_END);
    const unsigned long long file_size = (unsigned long long)ftell(fp);
    fseek(fp, 0, SEEK_SET);
    uint64_t header_size = 0;
    if (fread(&header_size, sizeof header_size, 1, fp) != 1)
        return fail(LLMB_ERR_IO, "%s: file shorter than the 8-byte header length", filename);
    if (header_size == 0 || header_size > file_size - 8 || header_size > (1ull << 30))
        return fail(LLMB_ERR_IO, "%s: header length runs past the end of the file", filename);
    std::vector<char> header((size_t)header_size);
    if (fread(header.data(), 1, header.size(), fp) != header.size())
        return fail(LLMB_ERR_IO, "%s: could not read the header", filename);

    std::vector<Entry> entries;
    if (!HeaderParser(header.data(), header.size()).parse(entries))
        return fail(LLMB_ERR_IO, "%s: Error parsing JSON", filename);

    const unsigned long long data_base = 8ull + header_size;
    llmb::ModelPriv *priv = llmb::model_priv(m);
    if (!priv) return fail(LLMB_ERR_NOMEM, "load_safetensor_weights: out of memory");
    int file_index = -1;
    for (const Entry &e : entries) {
        int needs_layer = 0;
        Tensor *t = slot_of_key(m, e.name, &needs_layer);
        if (!t) {
            if (needs_layer) return fail(LLMB_ERR_INVALID, "%s: layer index of '%s' is outside the model", filename, e.name.c_str());
            return fail(LLMB_ERR_INVALID, "%s: Component not allocated or not initialized properly: '%s'", filename,
                        e.name.c_str());
        }
        int dtype;
        if (e.dtype == "BF16") dtype = 0;
        else if (e.dtype == "F16") dtype = 1;
        else return fail(LLMB_ERR_UNSUPPORTED, "%s: dtype %s is neither BF16 nor F16", e.name.c_str(), e.dtype.c_str());
        if (e.shape.empty() || e.shape.size() > 2)
            return fail(LLMB_ERR_INVALID, "%s: tensor '%s' is not 1-D or 2-D", filename, e.name.c_str());
        unsigned long long count = 1;
        for (long long d : e.shape) {
            if (d <= 0 || d > 0x7fffffffLL) return fail(LLMB_ERR_INVALID, "%s: bad shape for '%s'", filename, e.name.c_str());
            count *= (unsigned long long)d;
        }
        if (count > 0x7fffffffULL) return fail(LLMB_ERR_INVALID, "%s: tensor '%s' too large", filename, e.name.c_str());
        if (e.end - e.begin != count * 2)
            return fail(LLMB_ERR_IO, "%s: data_offsets of '%s' do not match its shape", filename, e.name.c_str());
        if (data_base + e.end > file_size)
            return fail(LLMB_ERR_IO, "%s: payload of '%s' runs past the end of the file (truncated shard?)", filename,
                        e.name.c_str());

        free(t->ndim); free(t->mem_len); free(t->shape); free(t->bf16_tensor);
        t->bf16_tensor = nullptr;
        t->ndim = static_cast<int *>(malloc(sizeof(int)));
        t->mem_len = static_cast<int *>(malloc(sizeof(int)));
        t->shape = static_cast<int *>(malloc(sizeof(int) * 2));
        if (!t->ndim || !t->mem_len || !t->shape)
            return fail(LLMB_ERR_NOMEM, "Error: An Error Occurred while allocating memory for the component Tensor");
        *t->ndim = (int)e.shape.size();
        t->shape[0] = (int)e.shape[0];
        t->shape[1] = e.shape.size() > 1 ? (int)e.shape[1] : 1;
        *t->mem_len = (int)count;
        t->file_dtype = dtype;
        if (file_index < 0) {
            priv->files.push_back(filename);
            file_index = (int)priv->files.size() - 1;
        }
        llmb::TensorSource src;
        src.file = file_index;
        src.offset = data_base + e.begin;
        priv->sources[t] = src;
        if (!priv->streaming) {
            t->bf16_tensor = static_cast<uint16_t *>(malloc((size_t)count * 2));
            if (!t->bf16_tensor)
                return fail(LLMB_ERR_NOMEM, "Error: An Error Occurred while allocating memory for the component Tensor");
            if (fseek(fp, (long)(data_base + e.begin), SEEK_SET) != 0 ||
                fread(t->bf16_tensor, 2, (size_t)count, fp) != (size_t)count)
                return fail(LLMB_ERR_IO, "%s: short read on '%s'", filename, e.name.c_str());
        }
        t->loaded = 1;
    }
    return LLMB_OK;
}

extern "C" void load_safetensor_weights(Llama3 *m, const char *filename) {
    int rc = llama3_load_safetensors(m, filename);
    if (rc) {
        printf("%s\n", llmb_last_error());  // the reference prints and exits (safetensor.cu:20-23)
        exit(1);
    }
}
