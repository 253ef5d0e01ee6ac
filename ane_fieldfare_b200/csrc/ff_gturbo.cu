// Reader of an installed model's packed experts: `packed_experts/layout.json` and the layer files
// it names, straight into the HBM expert store.
//
// Host-only code (no kernels).  The checks are the reference's, rule for rule, with its messages:
//   * decode + structural validation of the layout
//     (Sources/ANEFieldfareImportedFormat/GTurboPackedExpertsLayoutV1.swift:65-162,
//      path rules Sources/ANEFieldfareImportedFormat/GTurboFormatV1.swift:52-80);
//   * the runtime's schema check of the routed experts against the model's shapes
//     (Sources/ANEFieldfareHotpath/Runtime/Inference/Model.swift:478-527);
//   * expert (layer, e) lives at physicalRank * expertStride of its layer file
//     (Sources/ANEFieldfareHotpath/Infrastructure/ModelIO/PackedExpertsLayout.swift:55-90,
//      Runtime/Inference/ModelExpertIO.swift:11-35).
// The reference maps the files and binds expert blobs by their physical offsets; here a layer's
// blobs are copied once into one device allocation in LOGICAL expert order (blob e at e * stride),
// which is what every kernel indexes, so physicalRank != expert costs nothing after the load.
#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "ff_internal.cuh"

namespace ff {
namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, true/false/null) -----------------

struct Json {
    enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
    bool boolean = false;
    bool isUnsigned = false;  // a non-negative integer that fits 64 bits
    uint64_t u = 0;
    double number = 0.0;
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json *get(const char *key) const {
        for (const auto &m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
};

class JsonParser {
public:
    JsonParser(const char *data, size_t size) : p_(data), end_(data + size) {}
    bool parse(Json *out, std::string *why) {
        if (!value(out, 0)) {
            *why = why_.empty() ? "malformed JSON" : why_;
            return false;
        }
        space();
        if (p_ != end_) {
            *why = "trailing characters after the JSON value";
            return false;
        }
        return true;
    }

private:
    const char *p_, *end_;
    std::string why_;
    void space() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    bool fail(const char *why) {
        if (why_.empty()) why_ = why;
        return false;
    }
    bool literal(const char *word) {
        const size_t n = strlen(word);
        if ((size_t)(end_ - p_) < n || memcmp(p_, word, n) != 0) return fail("unexpected token");
        p_ += n;
        return true;
    }
    bool string(std::string *out) {
        if (p_ >= end_ || *p_ != '"') return fail("expected a string");
        ++p_;
        out->clear();
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c == '\\') {
                if (p_ >= end_) return fail("unterminated escape");
                const char e = *p_++;
                switch (e) {
                    case '"': c = '"'; break;
                    case '\\': c = '\\'; break;
                    case '/': c = '/'; break;
                    case 'b': c = '\b'; break;
                    case 'f': c = '\f'; break;
                    case 'n': c = '\n'; break;
                    case 'r': c = '\r'; break;
                    case 't': c = '\t'; break;
                    case 'u': {
                        if (end_ - p_ < 4) return fail("short \\u escape");
                        unsigned code = 0;
                        for (int i = 0; i < 4; ++i) {
                            const char h = *p_++;
                            code <<= 4;
                            if (h >= '0' && h <= '9') code |= (unsigned)(h - '0');
                            else if (h >= 'a' && h <= 'f') code |= (unsigned)(h - 'a' + 10);
                            else if (h >= 'A' && h <= 'F') code |= (unsigned)(h - 'A' + 10);
                            else return fail("bad \\u escape");
                        }
                        // UTF-8 of the basic plane (surrogate pairs are not needed for file names here)
                        if (code < 0x80) out->push_back((char)code);
                        else if (code < 0x800) {
                            out->push_back((char)(0xC0 | (code >> 6)));
                            out->push_back((char)(0x80 | (code & 0x3F)));
                        } else {
                            out->push_back((char)(0xE0 | (code >> 12)));
                            out->push_back((char)(0x80 | ((code >> 6) & 0x3F)));
                            out->push_back((char)(0x80 | (code & 0x3F)));
                        }
                        continue;
                    }
                    default: return fail("unknown escape");
                }
            }
            out->push_back(c);
        }
        if (p_ >= end_) return fail("unterminated string");
        ++p_;
        return true;
    }
    bool number(Json *out) {
        const char *start = p_;
        if (p_ < end_ && *p_ == '-') ++p_;
        while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '+' || *p_ == '-')) ++p_;
        if (p_ == start) return fail("expected a number");
        const std::string text(start, p_);
        out->kind = Json::kNumber;
        out->number = strtod(text.c_str(), nullptr);
        out->isUnsigned = false;
        if (text.find_first_not_of("0123456789") == std::string::npos && text.size() <= 20) {
            errno = 0;
            const unsigned long long v = strtoull(text.c_str(), nullptr, 10);
            if (errno == 0) {
                out->isUnsigned = true;
                out->u = v;
            }
        }
        return true;
    }
    bool value(Json *out, int depth) {
        if (depth > 64) return fail("nesting too deep");
        space();
        if (p_ >= end_) return fail("unexpected end of input");
        switch (*p_) {
            case '{': {
                ++p_;
                out->kind = Json::kObject;
                space();
                if (p_ < end_ && *p_ == '}') {
                    ++p_;
                    return true;
                }
                for (;;) {
                    space();
                    std::string key;
                    if (!string(&key)) return false;
                    space();
                    if (p_ >= end_ || *p_ != ':') return fail("expected ':'");
                    ++p_;
                    out->members.emplace_back(std::move(key), Json());
                    if (!value(&out->members.back().second, depth + 1)) return false;
                    space();
                    if (p_ < end_ && *p_ == ',') {
                        ++p_;
                        continue;
                    }
                    if (p_ < end_ && *p_ == '}') {
                        ++p_;
                        return true;
                    }
                    return fail("expected ',' or '}'");
                }
            }
            case '[': {
                ++p_;
                out->kind = Json::kArray;
                space();
                if (p_ < end_ && *p_ == ']') {
                    ++p_;
                    return true;
                }
                for (;;) {
                    out->items.emplace_back();
                    if (!value(&out->items.back(), depth + 1)) return false;
                    space();
                    if (p_ < end_ && *p_ == ',') {
                        ++p_;
                        continue;
                    }
                    if (p_ < end_ && *p_ == ']') {
                        ++p_;
                        return true;
                    }
                    return fail("expected ',' or ']'");
                }
            }
            case '"': out->kind = Json::kString; return string(&out->text);
            case 't': out->kind = Json::kBool; out->boolean = true; return literal("true");
            case 'f': out->kind = Json::kBool; out->boolean = false; return literal("false");
            case 'n': out->kind = Json::kNull; return literal("null");
            default: return number(out);
        }
    }
};

// ---- the layout as the reference's wire structs hold it -----------------------------------------

struct SubTensor {
    uint64_t offset = 0, size = 0;
    std::string dtype;
    std::vector<uint32_t> shape;
    bool hasBits = false;
    int64_t bits = 0;
    bool operator==(const SubTensor &o) const {
        return offset == o.offset && size == o.size && dtype == o.dtype && shape == o.shape && hasBits == o.hasBits &&
               (!hasBits || bits == o.bits);
    }
};
struct Expert {
    bool hasExpert = false, hasPhysical = false;
    int64_t expert = 0, physicalRank = 0;
    uint64_t offset = 0, size = 0;
    std::map<std::string, SubTensor> tensors;
};
struct Layer {
    int64_t layer = 0;
    std::string file;
    std::vector<Expert> experts;
};
struct Layout {
    uint64_t expertStride = 0;
    int64_t numLayers = 0, expertsPerLayer = 0;
    std::vector<Layer> layers;
};

constexpr uint64_t kAlignmentBytes = 16384;  // GTurboFormatV1.alignmentBytes

std::string invalid(const std::string &field, const std::string &reason) { return field + ": " + reason; }

// A decode error in the reference's words ("packed_experts/layout.json: <what failed to decode>").
bool decode_error(std::string *why, const std::string &what) {
    *why = "packed_experts/layout.json: " + what;
    return false;
}
bool get_u64(const Json &obj, const char *key, uint64_t *out, std::string *why) {
    const Json *v = obj.get(key);
    if (!v) return decode_error(why, std::string("key \"") + key + "\" not found");
    if (v->kind != Json::kNumber || !v->isUnsigned) return decode_error(why, std::string("\"") + key + "\" is not an unsigned integer");
    *out = v->u;
    return true;
}
bool get_int(const Json &obj, const char *key, bool required, bool *present, int64_t *out, std::string *why) {
    const Json *v = obj.get(key);
    *present = v && v->kind != Json::kNull;
    if (!*present) return required ? decode_error(why, std::string("key \"") + key + "\" not found") : true;
    if (v->kind != Json::kNumber || v->number != (double)(int64_t)v->number)
        return decode_error(why, std::string("\"") + key + "\" is not an integer");
    *out = (int64_t)v->number;
    return true;
}

bool decode_layout(const Json &root, Layout *out, std::string *why) {
    if (root.kind != Json::kObject) return decode_error(why, "top level is not an object");
    bool present = false;
    if (!get_u64(root, "expertStride", &out->expertStride, why) ||
        !get_int(root, "numLayers", true, &present, &out->numLayers, why) ||
        !get_int(root, "expertsPerLayer", true, &present, &out->expertsPerLayer, why))
        return false;
    const Json *layers = root.get("layers");
    if (!layers || layers->kind != Json::kArray) return decode_error(why, "key \"layers\" not found");
    for (const Json &jl : layers->items) {
        if (jl.kind != Json::kObject) return decode_error(why, "a layer is not an object");
        Layer L;
        if (!get_int(jl, "layer", true, &present, &L.layer, why)) return false;
        const Json *file = jl.get("file");
        if (!file || file->kind != Json::kString) return decode_error(why, "key \"file\" not found");
        L.file = file->text;
        const Json *experts = jl.get("experts");
        if (!experts || experts->kind != Json::kArray) return decode_error(why, "key \"experts\" not found");
        for (const Json &je : experts->items) {
            if (je.kind != Json::kObject) return decode_error(why, "an expert is not an object");
            Expert E;
            if (!get_int(je, "expert", false, &E.hasExpert, &E.expert, why) ||
                !get_int(je, "physicalRank", false, &E.hasPhysical, &E.physicalRank, why) ||
                !get_u64(je, "offset", &E.offset, why) || !get_u64(je, "size", &E.size, why))
                return false;
            const Json *tensors = je.get("tensors");
            if (!tensors || tensors->kind != Json::kObject) return decode_error(why, "key \"tensors\" not found");
            for (const auto &m : tensors->members) {
                const Json &jt = m.second;
                if (jt.kind != Json::kObject) return decode_error(why, "a tensor is not an object");
                SubTensor t;
                if (!get_u64(jt, "offset", &t.offset, why) || !get_u64(jt, "size", &t.size, why)) return false;
                const Json *dtype = jt.get("dtype");
                if (!dtype || dtype->kind != Json::kString) return decode_error(why, "key \"dtype\" not found");
                t.dtype = dtype->text;
                const Json *shape = jt.get("shape");
                if (!shape || shape->kind != Json::kArray) return decode_error(why, "key \"shape\" not found");
                for (const Json &d : shape->items) {
                    if (d.kind != Json::kNumber || !d.isUnsigned || d.u > 0xFFFFFFFFull)
                        return decode_error(why, "a shape entry is not a 32-bit unsigned integer");
                    t.shape.push_back((uint32_t)d.u);
                }
                if (!get_int(jt, "bits", false, &t.hasBits, &t.bits, why)) return false;
                E.tensors[m.first] = t;
            }
            L.experts.push_back(std::move(E));
        }
        out->layers.push_back(std::move(L));
    }
    return true;
}

std::string lower_ascii(std::string s) {
    for (char &c : s)
        if (c >= 'A' && c <= 'Z') c = (char)(c - 'A' + 'a');
    return s;
}

// GTurboPathValidator.validateBasename (GTurboFormatV1.swift:58-79)
bool validate_basename(const std::string &name, const std::string &field, std::string *why) {
    if (name.empty() || name[0] == '/' || name.find('\0') != std::string::npos) {
        *why = invalid(field, "unsafe relative path");
        return false;
    }
    size_t start = 0;
    for (;;) {
        const size_t slash = name.find('/', start);
        const std::string part = name.substr(start, slash == std::string::npos ? std::string::npos : slash - start);
        if (part.empty() || part == "." || part == "..") {
            *why = invalid(field, "non-canonical path");
            return false;
        }
        if (slash == std::string::npos) break;
        start = slash + 1;
    }
    if (name.find('/') != std::string::npos) {
        *why = invalid(field, "expected basename");
        return false;
    }
    return true;
}

// GTurboV1StructuralValidator.validate (GTurboPackedExpertsLayoutV1.swift:75-162)
bool validate_structure(const Layout &layout, std::string *why) {
    if (layout.numLayers <= 0 || layout.expertsPerLayer <= 0 || layout.expertStride == 0 ||
        layout.expertStride % kAlignmentBytes != 0 || (int64_t)layout.layers.size() != layout.numLayers) {
        *why = invalid("layout", "invalid dimensions or stride");
        return false;
    }
    std::set<int64_t> layerIds;
    std::set<std::string> layerFiles;
    for (const Layer &layer : layout.layers) {
        const std::string tag = "layout.layers[" + std::to_string(layer.layer) + "]";
        if (layer.layer < 0 || layer.layer >= layout.numLayers || !layerIds.insert(layer.layer).second) {
            *why = invalid("layout.layers", "duplicate or invalid layer");
            return false;
        }
        if (!validate_basename(layer.file, tag + ".file", why)) return false;
        const std::string key = lower_ascii(layer.file);  // the case-insensitive file system key
        if (key == "layout.json") {
            *why = invalid(tag + ".file", "reserved packed-expert filename");
            return false;
        }
        if (!layerFiles.insert(key).second) {
            *why = invalid(tag + ".file", "duplicate layer filename");
            return false;
        }
        if ((int64_t)layer.experts.size() != layout.expertsPerLayer) {
            *why = invalid(tag + ".experts", "wrong expert count");
            return false;
        }
        size_t explicitIds = 0;
        for (const Expert &e : layer.experts) explicitIds += e.hasExpert ? 1 : 0;
        if (explicitIds != 0 && explicitIds != layer.experts.size()) {
            *why = invalid(tag + ".experts", "expert ids must be either all explicit or all positional");
            return false;
        }
        std::set<int64_t> logicalIds, physicalRanks;
        std::set<uint64_t> offsets;
        for (size_t position = 0; position < layer.experts.size(); ++position) {
            const Expert &e = layer.experts[position];
            const int64_t logical = e.hasExpert ? e.expert : (int64_t)position;
            const int64_t physical = e.hasPhysical ? e.physicalRank : logical;
            if (logical < 0 || logical >= layout.expertsPerLayer || physical < 0 || physical >= layout.expertsPerLayer ||
                !logicalIds.insert(logical).second || !physicalRanks.insert(physical).second ||
                !offsets.insert(e.offset).second) {
                *why = invalid(tag + ".experts", "duplicate or invalid expert mapping");
                return false;
            }
            const unsigned __int128 expected = (unsigned __int128)(uint64_t)physical * layout.expertStride;
            if (expected >> 64) {
                *why = "expert.offset: arithmetic overflow";
                return false;
            }
            const std::string etag = "expert[" + std::to_string(logical) + "]";
            if (e.offset != (uint64_t)expected || e.size != layout.expertStride) {
                *why = invalid(etag, "offset or size does not match physical rank");
                return false;
            }
            struct Range {
                uint64_t start, end;
                std::string name;
            };
            std::vector<Range> ranges;
            for (const auto &kv : e.tensors) {
                const SubTensor &t = kv.second;
                bool ok = (t.dtype == "U32" || t.dtype == "BF16") && !kv.first.empty() && t.size > 0 && !t.shape.empty() &&
                          (!t.hasBits || (t.bits > 0 && t.bits <= 32));
                for (uint32_t d : t.shape) ok = ok && d > 0;
                if (!ok) {
                    *why = invalid(etag + ".tensors." + kv.first, "invalid dtype or shape");
                    return false;
                }
                if (t.offset + t.size < t.offset) {
                    *why = "tensor." + kv.first + ".range: arithmetic overflow";
                    return false;
                }
                if (t.offset + t.size > e.size) {
                    *why = invalid(etag + ".tensors." + kv.first, "range exceeds expert blob");
                    return false;
                }
                ranges.push_back({t.offset, t.offset + t.size, kv.first});
            }
            std::sort(ranges.begin(), ranges.end(), [](const Range &a, const Range &b) {
                return a.start == b.start ? a.end < b.end : a.start < b.start;
            });
            for (size_t i = 0; i + 1 < ranges.size(); ++i)
                if (ranges[i].end > ranges[i + 1].start) {
                    *why = invalid(etag + ".tensors", "overlapping ranges " + ranges[i].name + " and " + ranges[i + 1].name);
                    return false;
                }
        }
    }
    return true;
}

// The runtime's schema check of the routed experts (Model.swift:478-527) for affine 4-bit weights
// in groups of 64; fills the nine offsets of every layer.
bool validate_schema(const Layout &layout, uint32_t d, uint32_t f, std::vector<FFExpertOffsets> *offsets, std::string *why) {
    const char *roles[3] = {"gate", "up", "down"};
    offsets->assign((size_t)layout.numLayers, FFExpertOffsets{});
    for (const Layer &layer : layout.layers) {
        const std::string tag = "routed layer " + std::to_string(layer.layer);
        if (layer.experts.empty()) {
            *why = tag + " has no experts";
            return false;
        }
        const Expert &reference = layer.experts.front();
        uint32_t *fields = &(*offsets)[(size_t)layer.layer].gateWOff;
        for (int m = 0; m < 3; ++m) {
            const uint64_t rows = m == 2 ? d : f, cols = m == 2 ? f : d;
            struct Want {
                std::string name, dtype;
                std::vector<uint32_t> shape;
                bool hasBits;
                uint64_t size, alignment;
            };
            const Want wants[3] = {
                {roles[m], "U32", {(uint32_t)rows, (uint32_t)(cols * 4 / 32)}, true, rows * cols / 2, 4},
                {std::string(roles[m]) + "_scales", "BF16", {(uint32_t)rows, (uint32_t)(cols / kGroup)}, false, rows * cols / kGroup * 2, 2},
                {std::string(roles[m]) + "_biases", "BF16", {(uint32_t)rows, (uint32_t)(cols / kGroup)}, false, rows * cols / kGroup * 2, 2},
            };
            for (int part = 0; part < 3; ++part) {
                const Want &w = wants[part];
                const auto it = reference.tensors.find(w.name);
                if (it == reference.tensors.end()) {
                    *why = tag + " is missing role " + w.name;
                    return false;
                }
                const SubTensor &t = it->second;
                const uint64_t end = t.offset + t.size;
                const bool bitsOk = w.hasBits ? (t.hasBits && t.bits == 4) : !t.hasBits;
                if (t.dtype != w.dtype || t.shape != w.shape || !bitsOk || t.size != w.size || t.offset % w.alignment != 0 ||
                    end < t.offset || end > reference.size || end > 0x100000000ull) {
                    *why = tag + " role " + w.name + " does not match the required schema";
                    return false;
                }
                for (size_t i = 1; i < layer.experts.size(); ++i) {
                    const auto other = layer.experts[i].tensors.find(w.name);
                    if (other == layer.experts[i].tensors.end() || !(other->second == t)) {
                        *why = tag + " role " + w.name + " metadata differs across experts";
                        return false;
                    }
                }
                fields[3 * m + part] = (uint32_t)t.offset;
            }
        }
    }
    return true;
}

bool read_file(const std::string &path, std::vector<char> *out, uint64_t maxBytes, std::string *why) {
    FILE *fh = fopen(path.c_str(), "rb");
    if (!fh) {
        *why = path + ": " + strerror(errno);
        return false;
    }
    fseek(fh, 0, SEEK_END);
    const long size = ftell(fh);
    fseek(fh, 0, SEEK_SET);
    if (size < 0 || (uint64_t)size > maxBytes) {
        fclose(fh);
        *why = path + ": file too large";
        return false;
    }
    out->resize((size_t)size);
    const size_t got = size ? fread(out->data(), 1, (size_t)size, fh) : 0;
    fclose(fh);
    if (got != (size_t)size) {
        *why = path + ": short read";
        return false;
    }
    return true;
}

bool load_layout(const char *modelDir, uint32_t d, uint32_t f, Layout *layout, std::vector<FFExpertOffsets> *offsets,
                 std::string *why) {
    if (d == 0 || f == 0 || d % kGroup || f % kGroup) {
        *why = "d and f must be non-zero multiples of the group size 64";
        return false;
    }
    std::vector<char> text;
    // PackedExpertsLayoutReader.defaultMaxBytes is 16 MiB for the reference's own models; a layout
    // of 30 layers x 128 experts is about 5 MB
    if (!read_file(std::string(modelDir) + "/packed_experts/layout.json", &text, 64ull << 20, why)) return false;
    Json root;
    JsonParser parser(text.data(), text.size());
    std::string parseWhy;
    if (!parser.parse(&root, &parseWhy)) return decode_error(why, parseWhy);
    return decode_layout(root, layout, why) && validate_structure(*layout, why) &&
           validate_schema(*layout, d, f, offsets, why);
}

}  // namespace
}  // namespace ff

using namespace ff;

extern "C" {

bool ff_gturbo_validate_layout(const char *modelDir, uint32_t d, uint32_t f, FFGTurboLayoutInfo *info,
                               const char **error) {
    if (error) *error = nullptr;
    if (!modelDir) return fail(error, "null argument");
    Layout layout;
    std::vector<FFExpertOffsets> offsets;
    std::string why;
    if (!load_layout(modelDir, d, f, &layout, &offsets, &why)) return fail(error, why);
    if (info) {
        info->expertStride = layout.expertStride;
        info->numLayers = (uint32_t)layout.numLayers;
        info->expertsPerLayer = (uint32_t)layout.expertsPerLayer;
        info->offsets = offsets[0];
        info->identityPlacement = 1;
        for (const Layer &layer : layout.layers)
            for (size_t position = 0; position < layer.experts.size(); ++position) {
                const Expert &e = layer.experts[position];
                const int64_t logical = e.hasExpert ? e.expert : (int64_t)position;
                if ((e.hasPhysical ? e.physicalRank : logical) != logical) info->identityPlacement = 0;
            }
    }
    return true;
}

bool ff_load_model_dir(FFContext *ctx, const char *modelDir, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !modelDir) return fail(error, "null argument");
    Layout layout;
    std::vector<FFExpertOffsets> offsets;
    std::string why;
    if (!load_layout(modelDir, ctx->cfg.d, ctx->cfg.f, &layout, &offsets, &why)) return fail(error, why);
    if ((uint64_t)layout.numLayers > ctx->cfg.layers)
        return fail(error, "the model has " + std::to_string(layout.numLayers) + " layers, the context holds " +
                               std::to_string(ctx->cfg.layers));
    if ((uint64_t)layout.expertsPerLayer != ctx->cfg.experts)
        return fail(error, "the model has " + std::to_string(layout.expertsPerLayer) + " experts per layer, the context expects " +
                               std::to_string(ctx->cfg.experts));
    const uint64_t stride = layout.expertStride;
    const uint64_t layerBytes = (uint64_t)layout.expertsPerLayer * stride;
    std::vector<char> file, ordered;
    for (const Layer &layer : layout.layers) {
        const std::string path = std::string(modelDir) + "/packed_experts/" + layer.file;
        if (!read_file(path, &file, layerBytes, &why)) return fail(error, why);
        // GTurboV1StructuralValidator.crossValidate: a layer file is exactly expertsPerLayer strides long
        if (file.size() != layerBytes)
            return fail(error, "manifest.files.packed_experts/" + layer.file + ": missing or wrong layer size");
        const char *bytes = file.data();
        bool identity = true;
        for (size_t position = 0; position < layer.experts.size(); ++position)
            identity = identity && layer.experts[position].offset == position * stride &&
                       (!layer.experts[position].hasExpert || layer.experts[position].expert == (int64_t)position);
        if (!identity) {
            // blob of logical expert e goes to e * stride: the order every kernel indexes
            ordered.resize(layerBytes);
            for (size_t position = 0; position < layer.experts.size(); ++position) {
                const Expert &e = layer.experts[position];
                const uint64_t logical = e.hasExpert ? (uint64_t)e.expert : position;
                memcpy(ordered.data() + logical * stride, file.data() + e.offset, stride);
            }
            bytes = ordered.data();
        }
        if (!ff_load_layer(ctx, (uint32_t)layer.layer, bytes, layerBytes, (uint32_t)layout.expertsPerLayer, stride,
                           &offsets[(size_t)layer.layer], error))
            return false;
    }
    return true;
}

}  // extern "C"
