// Minimal FlatBuffers reader and writer for the tinynn model format
// (root table MegCC.Model of runtime/schema/model.fbs in the reference). Field numbers
// below are the declaration order of that schema; the bytes are interchangeable with
// files written by the reference's exporter (compiler/lib/Target/TinyNN/exporter.cpp).
//
// The reader bounds-checks every access and reports failure instead of reading outside
// the buffer, so a truncated or corrupt model turns into TinyNN_ERROR_MODEL_PARSE.
#pragma once
#include <stdint.h>
#include <string.h>

#include <memory>
#include <string>
#include <vector>

namespace tinynn_fb {

// ---- schema constants ---------------------------------------------------------------------
enum DTypeEnum : int8_t {
    Float32 = 0, Float16 = 1, Int32 = 2, Int8 = 3, Int16 = 4, Uint8 = 5,
    QInt8 = 100, QInt32 = 101, QUint8 = 102
};
enum Format : int8_t { NCHW = 0, NHWC = 1, NCHW4 = 2, NCHW8 = 3, OIHW = 4 };
// "only add new device at the end" (model.fbs:39): CUDA_SM100 follows WEB_ASSEMBLY
enum Device : int8_t {
    BARE_METAL = 0, ARM64 = 1, ARM32 = 2, ARM64_V82 = 3, ARM32_V82 = 4, OPENCL_MALI = 5,
    WEB_ASSEMBLY = 6, CUDA_SM100 = 7
};
enum TensorType : int8_t { TENSOR = 0, WEIGHT = 1 };
enum InstructionTag : uint8_t { INST_NONE = 0, INST_OPR = 1, INST_MEM_FORWARD = 4 };

namespace field {
enum Model { M_weight_pool = 0, M_device_models = 1, M_const_shape = 2, M_name = 3, M_model_id = 4 };
enum DeviceModel {
    D_device = 0, D_tensor_pool = 1, D_instructions_type = 2, D_instructions = 3,
    D_tensor_memory = 4, D_inputs = 5, D_outputs = 6, D_weight_outputs = 7,
    D_weight_outputs_name = 8
};
enum Tensor { T_dtype = 0, T_layout = 1, T_offset = 2, T_dynamic = 3, T_use_count = 4, T_name = 5 };
enum DType { DT_type = 0, DT_param = 1 };
enum DTypeParam { DP_scale = 0, DP_zero_point = 1 };
enum Layout { L_dims = 0, L_stride = 1, L_format = 2 };
enum Weight {
    W_dtype = 0, W_layout = 1, W_use_count = 2, W_data = 3, W_name = 4, W_checksum = 5,
    W_compressed = 6
};
enum Opr {
    O_name = 0, O_type = 1, O_inputs = 2, O_input_types = 3, O_outputs = 4, O_workspace = 5,
    O_init_id = 6, O_kernel_id = 7, O_workspace_id = 8, O_deduce_id = 9
};
enum Workspace { WS_size = 0, WS_offset = 1 };
enum MemForward { MF_input = 0, MF_output = 1, MF_offset = 2, MF_type = 3 };
}  // namespace field

// ---- reader -------------------------------------------------------------------------------
struct Buffer {
    const uint8_t* data = nullptr;
    size_t size = 0;
    mutable bool failed = false;

    bool in(size_t pos, size_t len) const {
        if (pos > size || len > size - pos) {
            failed = true;
            return false;
        }
        return true;
    }
    template <class T>
    T rd(size_t pos) const {
        T v{};
        if (in(pos, sizeof(T)))
            memcpy(&v, data + pos, sizeof(T));
        return v;
    }
};

struct Vec {
    const Buffer* b = nullptr;
    size_t pos = 0;  // position of the first element
    uint32_t len = 0;
    explicit operator bool() const { return b != nullptr; }
    template <class T>
    T at(uint32_t i) const {
        return i < len ? b->rd<T>(pos + (size_t)i * sizeof(T)) : T{};
    }
    const uint8_t* bytes() const { return b && b->in(pos, len) ? b->data + pos : nullptr; }
};

struct Table {
    const Buffer* b = nullptr;
    size_t pos = 0;
    explicit operator bool() const { return b != nullptr; }

    size_t field_pos(int id) const {
        if (!b)
            return 0;
        const int32_t so = b->rd<int32_t>(pos);
        const long long vt = (long long)pos - so;
        if (vt < 0 || !b->in((size_t)vt, 4))
            return 0;
        const uint16_t vsize = b->rd<uint16_t>((size_t)vt);
        const size_t slot = 4 + 2 * (size_t)id;
        if (slot + 2 > vsize)
            return 0;
        const uint16_t off = b->rd<uint16_t>((size_t)vt + slot);
        return off ? pos + off : 0;
    }
    template <class T>
    T scalar(int id, T dflt) const {
        const size_t p = field_pos(id);
        return p ? b->rd<T>(p) : dflt;
    }
    size_t indirect(int id) const {
        const size_t p = field_pos(id);
        if (!p)
            return 0;
        const uint32_t off = b->rd<uint32_t>(p);
        if (off == 0 || !b->in(p + off, 4)) {
            b->failed = true;
            return 0;
        }
        return p + off;
    }
    Table table(int id) const {
        const size_t p = indirect(id);
        return p ? Table{b, p} : Table{};
    }
    Vec vec(int id, size_t elem_size) const {
        const size_t p = indirect(id);
        if (!p)
            return Vec{};
        const uint32_t len = b->rd<uint32_t>(p);
        if (!b->in(p + 4, (size_t)len * elem_size))
            return Vec{};
        return Vec{b, p + 4, len};
    }
    // element i of a vector of tables
    static Table elem(const Vec& v, uint32_t i) {
        if (!v || i >= v.len)
            return Table{};
        const size_t p = v.pos + (size_t)i * 4;
        const uint32_t off = v.b->rd<uint32_t>(p);
        if (off == 0 || !v.b->in(p + off, 4)) {
            v.b->failed = true;
            return Table{};
        }
        return Table{v.b, p + off};
    }
    bool str(int id, std::string* out) const {
        const Vec v = vec(id, 1);
        if (!v)
            return false;
        const uint8_t* s = v.bytes();
        if (!s)
            return false;
        out->assign((const char*)s, v.len);
        return true;
    }
};

inline Table root(const Buffer& b) {
    if (b.size < 8)
        return Table{};
    const uint32_t off = b.rd<uint32_t>(0);
    if (off < 4 || !b.in(off, 4))
        return Table{};
    return Table{&b, off};
}

// ---- writer -------------------------------------------------------------------------------
// A tree of nodes serialised front to back: a table is followed (not preceded) by the
// objects it points to, so every uoffset is positive as the format requires.
struct Node;
using NodeP = std::shared_ptr<Node>;

struct Node {
    enum Kind { TABLE, VEC_SCALAR, VEC_TABLE, STRING } kind = TABLE;
    // TABLE
    struct Field {
        int id;
        int size;         // 1,2,4,8 for scalars; 4 for references
        uint64_t scalar;  // raw little-endian bits
        NodeP ref;        // non-null: offset field
    };
    std::vector<Field> fields;
    // VEC_SCALAR / STRING
    std::vector<uint8_t> bytes;
    int elem_size = 1;
    // VEC_TABLE
    std::vector<NodeP> elems;

    template <class T>
    Node& add(int id, T v) {
        uint64_t bits = 0;
        memcpy(&bits, &v, sizeof(T));
        fields.push_back({id, (int)sizeof(T), bits, nullptr});
        return *this;
    }
    Node& add_ref(int id, NodeP n) {
        if (n)
            fields.push_back({id, 4, 0, std::move(n)});
        return *this;
    }
};

inline NodeP make_table() {
    return std::make_shared<Node>();
}
inline NodeP make_string(const std::string& s) {
    auto n = std::make_shared<Node>();
    n->kind = Node::STRING;
    n->bytes.assign(s.begin(), s.end());
    return n;
}
template <class T>
NodeP make_vec(const std::vector<T>& v) {
    auto n = std::make_shared<Node>();
    n->kind = Node::VEC_SCALAR;
    n->elem_size = sizeof(T);
    n->bytes.resize(v.size() * sizeof(T));
    if (!v.empty())
        memcpy(n->bytes.data(), v.data(), n->bytes.size());
    return n;
}
inline NodeP make_bytes(const void* p, size_t len) {
    auto n = std::make_shared<Node>();
    n->kind = Node::VEC_SCALAR;
    n->elem_size = 1;
    n->bytes.assign((const uint8_t*)p, (const uint8_t*)p + len);
    return n;
}
inline NodeP make_table_vec(std::vector<NodeP> elems) {
    auto n = std::make_shared<Node>();
    n->kind = Node::VEC_TABLE;
    n->elems = std::move(elems);
    return n;
}

class Writer {
public:
    std::vector<uint8_t> finish(const NodeP& root_table) {
        out_.assign(8, 0);  // root uoffset + padding keeps 8-byte alignment
        const size_t pos = emit(root_table);
        put<uint32_t>(0, (uint32_t)pos);
        return out_;
    }

private:
    std::vector<uint8_t> out_;

    void align(size_t a) {
        while (out_.size() % a)
            out_.push_back(0);
    }
    template <class T>
    void put(size_t pos, T v) {
        memcpy(out_.data() + pos, &v, sizeof(T));
    }
    template <class T>
    void push(T v) {
        const size_t p = out_.size();
        out_.resize(p + sizeof(T));
        put<T>(p, v);
    }

    // returns the position the object is referenced by
    size_t emit(const NodeP& n) {
        switch (n->kind) {
            case Node::STRING: {
                align(4);
                const size_t p = out_.size();
                push<uint32_t>((uint32_t)n->bytes.size());
                out_.insert(out_.end(), n->bytes.begin(), n->bytes.end());
                out_.push_back(0);
                return p;
            }
            case Node::VEC_SCALAR: {
                // the element block must be aligned to the element size; the length word
                // sits right before it
                const size_t a = n->elem_size > 4 ? (size_t)n->elem_size : 4;
                while ((out_.size() + 4) % a)
                    out_.push_back(0);
                const size_t p = out_.size();
                push<uint32_t>((uint32_t)(n->bytes.size() / n->elem_size));
                out_.insert(out_.end(), n->bytes.begin(), n->bytes.end());
                return p;
            }
            case Node::VEC_TABLE: {
                align(4);
                const size_t p = out_.size();
                push<uint32_t>((uint32_t)n->elems.size());
                const size_t slots = out_.size();
                out_.resize(slots + 4 * n->elems.size(), 0);
                for (size_t i = 0; i < n->elems.size(); ++i) {
                    const size_t child = emit(n->elems[i]);
                    const size_t slot = slots + 4 * i;
                    put<uint32_t>(slot, (uint32_t)(child - slot));
                }
                return p;
            }
            case Node::TABLE:
            default:
                return emit_table(n);
        }
    }

    size_t emit_table(const NodeP& n) {
        int max_id = -1;
        for (auto& f : n->fields)
            max_id = f.id > max_id ? f.id : max_id;
        // inline layout: soffset, then fields largest first so natural alignment holds
        std::vector<const Node::Field*> order;
        for (int sz : {8, 4, 2, 1})
            for (auto& f : n->fields)
                if (f.size == sz)
                    order.push_back(&f);
        std::vector<uint16_t> offs(max_id + 1, 0);
        size_t tsize = 4;
        bool has8 = false;
        for (auto* f : order) {
            has8 |= f->size == 8;
            while (tsize % f->size)
                ++tsize;
            offs[f->id] = (uint16_t)tsize;
            tsize += f->size;
        }
        const size_t vsize = 4 + 2 * (size_t)(max_id + 1);
        // place the vtable immediately before the table; the table start (+4 when it holds
        // 8-byte scalars, since those sit at offset 8 after the soffset and one 4-byte pad)
        // must keep the scalar alignment
        align(has8 ? 8 : 4);
        while ((out_.size() + vsize) % (has8 ? 8 : 4))
            out_.push_back(0);
        const size_t vt = out_.size();
        push<uint16_t>((uint16_t)vsize);
        push<uint16_t>((uint16_t)tsize);
        for (int i = 0; i <= max_id; ++i)
            push<uint16_t>(offs[i]);
        const size_t tpos = out_.size();
        out_.resize(tpos + tsize, 0);
        put<int32_t>(tpos, (int32_t)(tpos - vt));
        for (auto* f : order) {
            if (!f->ref)
                memcpy(out_.data() + tpos + offs[f->id], &f->scalar, f->size);
        }
        for (auto* f : order) {
            if (f->ref) {
                const size_t child = emit(f->ref);
                const size_t slot = tpos + offs[f->id];
                put<uint32_t>(slot, (uint32_t)(child - slot));
            }
        }
        return tpos;
    }
};

}  // namespace tinynn_fb
