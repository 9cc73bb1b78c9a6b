// Stand-alone evaluator behind cb_model_capi.h: parses a `.cbm` file (magic "CBM1", size, FlatBuffers core with the model
// trees, then the CTR value tables; layout of catboost/libs/model/flatbuffers/model.fbs, features.fbs, ctr_data.fbs and
// catboost/libs/model/model.cpp:1113-1230) and applies it on the host.
//
// Evaluation works on blocks of documents.  Every feature the model tests (numerical, one-hot categorical, CTR) is first
// turned into one byte per document, the number of borders the value exceeds (or 1 + the index of the matching one-hot
// value), so that a split is a byte compare and an oblivious tree is `depth` passes of compare-shift-or over the block,
// which the compiler vectorises.  A feature with more than 254 borders takes several byte columns.
#include "cb_model_capi.h"

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "cb_cityhash.h"

namespace {

thread_local std::string g_error;

[[noreturn]] void fail(const std::string& msg) { throw std::runtime_error(msg); }

// ---- FlatBuffers reading (bounds-checked; no generated code) ---------------------------------------------------------
struct Buf {
    const uint8_t* p;
    size_t n;
    template <class T> T rd(size_t pos) const {
        if (pos + sizeof(T) > n || pos + sizeof(T) < pos) fail("model file is truncated");
        T v;
        std::memcpy(&v, p + pos, sizeof(T));
        return v;
    }
};

struct Table {
    Buf b{nullptr, 0};
    size_t pos = 0;
    bool ok = false;

    static Table root(Buf b) { return Table{b, (size_t)b.rd<uint32_t>(0), true}; }
    size_t field(int id) const {
        const size_t vt = pos - (size_t)(int64_t)b.rd<int32_t>(pos);
        const size_t vt_size = b.rd<uint16_t>(vt);
        const size_t slot = 4 + 2 * (size_t)id;
        if (slot + 2 > vt_size) return 0;
        return b.rd<uint16_t>(vt + slot);
    }
    template <class T> T scalar(int id, T dflt) const {
        const size_t off = field(id);
        return off ? b.rd<T>(pos + off) : dflt;
    }
    size_t indirect(int id) const {
        const size_t off = field(id);
        if (!off) return 0;
        return pos + off + b.rd<uint32_t>(pos + off);
    }
    Table table(int id) const {
        const size_t t = indirect(id);
        return t ? Table{b, t, true} : Table{};
    }
    // raw view of a vector of fixed-size elements: element count and the position of element 0
    size_t vec(int id, size_t elem, size_t* data) const {
        const size_t v = indirect(id);
        if (!v) { *data = 0; return 0; }
        const size_t len = b.rd<uint32_t>(v);
        if (len && (v + 4 + len * elem > b.n)) fail("model file is truncated");
        *data = v + 4;
        return len;
    }
    template <class T> std::vector<T> vector(int id) const {
        size_t data;
        const size_t len = vec(id, sizeof(T), &data);
        std::vector<T> out(len);
        if (len) std::memcpy(out.data(), b.p + data, len * sizeof(T));
        return out;
    }
    std::string string(int id) const {
        size_t data;
        const size_t len = vec(id, 1, &data);
        return std::string((const char*)b.p + data, len);
    }
    std::vector<Table> tables(int id) const {
        size_t data;
        const size_t len = vec(id, 4, &data);
        std::vector<Table> out;
        for (size_t k = 0; k < len; ++k) {
            const size_t at = data + 4 * k;
            out.push_back(Table{b, at + b.rd<uint32_t>(at), true});
        }
        return out;
    }
    std::vector<std::string> strings(int id) const {
        size_t data;
        const size_t len = vec(id, 4, &data);
        std::vector<std::string> out;
        for (size_t k = 0; k < len; ++k) {
            const size_t at = data + 4 * k;
            const size_t s = at + b.rd<uint32_t>(at);
            const size_t sl = b.rd<uint32_t>(s);
            if (s + 4 + sl > b.n) fail("model file is truncated");
            out.emplace_back((const char*)b.p + s + 4, sl);
        }
        return out;
    }
};

// ---- the parsed model ------------------------------------------------------------------------------------------------
enum Kind : uint8_t { K_FLOAT = 0, K_ONEHOT = 1, K_CTR = 2 };
enum CtrType { CT_BORDERS = 0, CT_BUCKETS, CT_BIN_MEAN, CT_FLOAT_MEAN, CT_COUNTER, CT_FREQ };

struct FloatFeature {
    int index = -1, flat = -1;
    std::vector<float> borders;
    bool nan_is_max = false;
    std::string name;
};
struct CatFeature {
    int index = -1, flat = -1;
    std::string name;
};
struct OneHot {
    int cat_index = -1;            // position in the model's categorical feature list
    std::vector<uint32_t> values;
};
#pragma pack(push, 1)
struct Bucket { uint64_t hash; uint32_t index; };
#pragma pack(pop)
struct CtrTable {
    std::vector<int> cats;
    int type = 0;
    std::vector<Bucket> buckets;   // open addressing, 2^k entries, empty = all ones, linear probing
    std::vector<uint8_t> blob;
    int denominator = 0, n_classes = 0;
};
struct CtrFeature {
    int table = -1;                // index into Model::ctr_tables, -1 = no statistics stored
    std::vector<int> cat_pos;      // positions in the model's categorical feature list
    int type = 0, target_border = 0;
    float prior_num = 0, prior_denom = 1, shift = 0, scale = 1;
    std::vector<float> borders;
};
// one byte column of the block: which source it quantises and which of its borders
struct Column {
    Kind kind;
    int src;                       // float feature / one-hot / ctr list position
    int first;                     // first border (value) this column covers
    int count;                     // how many of them (<= 254)
};
// a split as the trees address it
struct BinSplit {
    int column;
    uint8_t threshold;             // numerical, ctr: bin >= threshold;  one-hot: bin == threshold
    uint8_t equal;
};

struct Model {
    int dims = 1;
    std::vector<FloatFeature> floats;
    std::vector<CatFeature> cats;
    std::vector<OneHot> onehots;
    std::vector<CtrTable> ctr_tables;
    std::vector<CtrFeature> ctrs;
    std::vector<Column> columns;
    std::vector<BinSplit> splits;
    // oblivious trees
    std::vector<int> tree_splits, tree_sizes, tree_starts;
    std::vector<size_t> tree_leaf_start;       // first leaf of every oblivious tree (in leaves, not values)
    // non-symmetric trees
    std::vector<uint16_t> step_left, step_right;
    std::vector<uint32_t> node_to_leaf;
    bool oblivious = true;
    std::vector<double> leaf_values;
    double scale = 1.0;
    std::vector<double> bias;
    std::map<std::string, std::string> info;
    int prediction_type = APT_RAW_FORMULA_VAL;
    int flat_size = 0;                          // 1 + the largest flat feature index
    size_t n_trees() const { return tree_sizes.size(); }
};

int cat_position(const Model& m, int cat_index) {
    for (size_t k = 0; k < m.cats.size(); ++k)
        if (m.cats[k].index == cat_index) return (int)k;
    fail("the model refers to a categorical feature it does not describe");
}

void read_ctr_base(const Table& base, std::vector<int>* cats, int* type) {
    const Table comb = base.table(0);
    if (comb.ok) {
        *cats = comb.vector<int>(0);
        size_t d;
        if (comb.vec(1, 1, &d) || comb.vec(2, 1, &d))
            fail("CTR projections over binarised numerical or one-hot features are not supported by this evaluator");
    }
    *type = base.scalar<int8_t>(1, 0);
}

void parse_ctr_tables(Model& m, const uint8_t* p, size_t n) {
    Buf b{p, n};
    const uint32_t count = b.rd<uint32_t>(0);
    size_t pos = 4;
    for (uint32_t k = 0; k < count; ++k) {
        const uint32_t size = b.rd<uint32_t>(pos);
        pos += 4;
        if (pos + size > n) fail("model file is truncated (CTR tables)");
        const Table t = Table::root(Buf{p + pos, size});
        pos += size;
        CtrTable ct;
        read_ctr_base(t.table(0), &ct.cats, &ct.type);
        size_t data;
        const size_t raw = t.vec(1, 1, &data);
        if (raw % sizeof(Bucket)) fail("malformed CTR hash index");
        ct.buckets.resize(raw / sizeof(Bucket));
        if (raw) std::memcpy(ct.buckets.data(), t.b.p + data, raw);
        if (ct.buckets.size() & (ct.buckets.size() - 1)) fail("CTR hash index size is not a power of two");
        ct.blob = t.vector<uint8_t>(2);
        ct.denominator = t.scalar<int32_t>(3, 0);
        ct.n_classes = t.scalar<int32_t>(4, 0);
        m.ctr_tables.push_back(std::move(ct));
    }
}

void parse_model(Model& m, const uint8_t* data, size_t size) {
    if (size < 8 || std::memcmp(data, "CBM1", 4) != 0) fail("not a cbm file: bad magic");
    uint64_t core_size;
    uint32_t s32;
    std::memcpy(&s32, data + 4, 4);
    size_t pos = 8;
    core_size = s32;
    if (s32 == 0xFFFFFFFFu) {
        if (size < 16) fail("model file is truncated");
        std::memcpy(&core_size, data + 8, 8);
        pos = 16;
    }
    if (pos + core_size > size) fail("model file is truncated");
    const Table core = Table::root(Buf{data + pos, (size_t)core_size});
    const uint8_t* rest = data + pos + core_size;
    const size_t rest_size = size - pos - (size_t)core_size;
    if (core.string(0) != "FlabuffersModel_v1") fail("unsupported model format '" + core.string(0) + "'");
    const Table mt = core.table(1);
    if (!mt.ok) fail("the model file holds no trees");
    for (const Table& kv : core.tables(2)) m.info[kv.string(0)] = kv.string(1);
    {
        size_t d;
        if (mt.vec(12, 4, &d) || mt.vec(13, 4, &d) || mt.vec(18, 4, &d))
            fail("the model uses text or embedding features, which this evaluator does not compute");
    }
    m.dims = std::max(1, (int)mt.scalar<int32_t>(0, 1));
    m.tree_splits = mt.vector<int>(1);
    m.tree_sizes = mt.vector<int>(2);
    m.tree_starts = mt.vector<int>(3);
    for (const Table& c : mt.tables(4)) {
        CatFeature cf;
        cf.index = c.scalar<int32_t>(0, -1);
        cf.flat = c.scalar<int32_t>(1, -1);
        cf.name = c.string(2);
        m.cats.push_back(cf);
    }
    for (const Table& f : mt.tables(5)) {
        FloatFeature ff;
        ff.index = f.scalar<int32_t>(1, -1);
        ff.flat = f.scalar<int32_t>(2, -1);
        ff.borders = f.vector<float>(3);
        ff.name = f.string(4);
        ff.nan_is_max = f.scalar<int8_t>(5, 0) == 2;
        m.floats.push_back(std::move(ff));
    }
    std::sort(m.floats.begin(), m.floats.end(), [](const FloatFeature& a, const FloatFeature& b) { return a.index < b.index; });
    std::sort(m.cats.begin(), m.cats.end(), [](const CatFeature& a, const CatFeature& b) { return a.index < b.index; });
    for (const Table& o : mt.tables(6)) {
        OneHot oh;
        oh.cat_index = cat_position(m, o.scalar<int32_t>(0, -1));
        for (int v : o.vector<int>(1)) oh.values.push_back((uint32_t)v);
        m.onehots.push_back(std::move(oh));
    }
    const std::vector<Table> ctr_feats = mt.tables(7);
    if (!ctr_feats.empty()) {
        const std::vector<std::string> parts = core.strings(3);
        if (!parts.empty() && parts[0] == "static_provider_v1") parse_ctr_tables(m, rest, rest_size);
        for (const Table& t : ctr_feats) {
            const Table ctr = t.table(0);
            if (!ctr.ok) fail("malformed CTR feature");
            CtrFeature cf;
            std::vector<int> cats;
            read_ctr_base(ctr.table(0), &cats, &cf.type);
            for (int c : cats) cf.cat_pos.push_back(cat_position(m, c));
            cf.target_border = ctr.scalar<int32_t>(1, 0);
            cf.prior_num = ctr.scalar<float>(2, 0.0f);
            cf.prior_denom = ctr.scalar<float>(3, 1.0f);
            cf.shift = ctr.scalar<float>(4, 0.0f);
            cf.scale = ctr.scalar<float>(5, 1.0f);
            cf.borders = t.vector<float>(1);
            for (size_t k = 0; k < m.ctr_tables.size(); ++k)
                if (m.ctr_tables[k].cats == cats && m.ctr_tables[k].type == cf.type) cf.table = (int)k;
            m.ctrs.push_back(std::move(cf));
        }
    }
    // byte columns and the split list, in the order the trees number their splits: numerical features with their borders,
    // then one-hot values, then CTR borders
    auto add_source = [&](Kind kind, int src, int total, bool equal) {
        for (int first = 0; first < total || first == 0; first += 254) {
            const int cnt = std::min(254, total - first);
            if (cnt <= 0) break;
            m.columns.push_back(Column{kind, src, first, cnt});
            for (int j = 0; j < cnt; ++j)
                m.splits.push_back(BinSplit{(int)m.columns.size() - 1, (uint8_t)(j + 1), (uint8_t)equal});
        }
    };
    for (size_t k = 0; k < m.floats.size(); ++k) add_source(K_FLOAT, (int)k, (int)m.floats[k].borders.size(), false);
    for (size_t k = 0; k < m.onehots.size(); ++k) add_source(K_ONEHOT, (int)k, (int)m.onehots[k].values.size(), true);
    for (size_t k = 0; k < m.ctrs.size(); ++k) add_source(K_CTR, (int)k, (int)m.ctrs[k].borders.size(), false);

    m.leaf_values = mt.vector<double>(8);
    {
        size_t d;
        const size_t steps = mt.vec(10, 4, &d);
        m.oblivious = steps == 0;
        for (size_t k = 0; k < steps; ++k) {
            m.step_left.push_back(mt.b.rd<uint16_t>(d + 4 * k));
            m.step_right.push_back(mt.b.rd<uint16_t>(d + 4 * k + 2));
        }
    }
    m.node_to_leaf = mt.vector<uint32_t>(11);
    m.scale = mt.scalar<double>(14, 1.0);
    m.bias = mt.vector<double>(16);
    if (m.bias.empty()) m.bias.assign(m.dims, mt.scalar<double>(15, 0.0));
    if ((int)m.bias.size() != m.dims) fail("bias size differs from the model dimension");
    if (m.tree_starts.size() != m.tree_sizes.size()) {
        m.tree_starts.assign(m.tree_sizes.size(), 0);
        for (size_t k = 1; k < m.tree_sizes.size(); ++k) m.tree_starts[k] = m.tree_starts[k - 1] + m.tree_sizes[k - 1];
    }
    for (size_t k = 0; k < m.tree_splits.size(); ++k) {
        if (!m.oblivious && k < m.step_left.size() && m.step_left[k] == 0 && m.step_right[k] == 0) continue;   // leaf node
        const int s = m.tree_splits[k];
        if (s < 0 || (size_t)s >= m.splits.size()) fail("a tree refers to a split the model does not describe");
    }
    size_t leaves = 0;
    for (size_t t = 0; t < m.n_trees(); ++t) {
        const int sz = m.tree_sizes[t];
        if (sz < 0 || (size_t)m.tree_starts[t] + sz > m.tree_splits.size()) fail("malformed tree table");
        if (m.oblivious) {
            if (sz > 30) fail("tree depth above 30");
            m.tree_leaf_start.push_back(leaves);
            leaves += (size_t)1 << sz;
        }
    }
    if (m.oblivious && leaves * m.dims > m.leaf_values.size()) fail("leaf value table is too short");
    if (!m.oblivious) {
        if (m.node_to_leaf.size() < m.tree_splits.size() || m.step_left.size() < m.tree_splits.size())
            fail("malformed non-symmetric tree table");
    }
    for (const auto& f : m.floats) m.flat_size = std::max(m.flat_size, f.flat + 1);
    for (const auto& c : m.cats) m.flat_size = std::max(m.flat_size, c.flat + 1);
}


// ---- evaluation ------------------------------------------------------------------------------------------------------
constexpr int BLOCK = 128;
constexpr uint64_t MAGIC_MULT = 0x4906ba494954cb65ULL;

// how a caller hands over its documents
struct Input {
    enum Layout { FLAT, FLAT_TRANSPOSED, SPLIT_STRINGS, SPLIT_HASHES } layout = FLAT;
    const float* const* floats = nullptr;     // [doc][feature] (FLAT_TRANSPOSED: [feature][doc])
    size_t floats_size = 0;
    const char* const* const* cat_strings = nullptr;
    const int* const* cat_hashes = nullptr;
    size_t cats_size = 0;
};

inline float float_value(const Model& m, const Input& in, const FloatFeature& f, size_t doc) {
    switch (in.layout) {
        case Input::FLAT: return in.floats[doc][f.flat];
        case Input::FLAT_TRANSPOSED: return in.floats[f.flat][doc];
        default: return in.floats[doc][f.index];
    }
    (void)m;
}

inline uint32_t cat_value(const Input& in, const CatFeature& c, size_t doc) {
    switch (in.layout) {
        case Input::FLAT: { uint32_t v; std::memcpy(&v, &in.floats[doc][c.flat], 4); return v; }
        case Input::FLAT_TRANSPOSED: { uint32_t v; std::memcpy(&v, &in.floats[c.flat][doc], 4); return v; }
        case Input::SPLIT_HASHES: return (uint32_t)in.cat_hashes[doc][c.index];
        default: {
            const char* s = in.cat_strings[doc][c.index];
            return (uint32_t)(city1::hash(s, std::strlen(s)) & 0xffffffffULL);
        }
    }
}

void check_input(const Model& m, const Input& in) {
    const bool flat = in.layout == Input::FLAT || in.layout == Input::FLAT_TRANSPOSED;
    size_t need_f = 0, need_c = 0;
    // only the features that the trees can reach have to be present
    for (const auto& f : m.floats)
        if (!f.borders.empty()) need_f = std::max(need_f, (size_t)(flat ? f.flat : f.index) + 1);
    bool cats_used = !m.onehots.empty() || !m.ctrs.empty();
    if (cats_used)
        for (const auto& c : m.cats) {
            if (flat) need_f = std::max(need_f, (size_t)c.flat + 1);
            else need_c = std::max(need_c, (size_t)c.index + 1);
        }
    if (in.floats_size < need_f)
        fail("the model needs " + std::to_string(need_f) + " feature values per document, got " + std::to_string(in.floats_size));
    if (in.cats_size < need_c)
        fail("the model needs " + std::to_string(need_c) + " categorical values per document, got " + std::to_string(in.cats_size));
    if (need_f && !in.floats) fail("feature pointer is null");
    if (need_c && !in.cat_strings && !in.cat_hashes) fail("categorical feature pointer is null");
}

float ctr_value(const Model& m, const CtrFeature& cf, const uint32_t* cat_hashes /* [cats][BLOCK] */, int d) {
    uint64_t h = 0;
    for (int pos : cf.cat_pos) {
        const uint64_t b = (uint64_t)(int64_t)(int32_t)cat_hashes[(size_t)pos * BLOCK + d];
        h = MAGIC_MULT * (h + MAGIC_MULT * b);
    }
    double good = 0.0, total = 0.0;
    int denominator = 0;
    if (cf.table >= 0) {
        const CtrTable& t = m.ctr_tables[cf.table];
        denominator = t.denominator;
        if (!t.buckets.empty()) {
            const size_t mask = t.buckets.size() - 1;
            size_t z = (size_t)h & mask;
            for (size_t probes = 0; probes <= mask; ++probes, z = (z + 1) & mask) {
                const Bucket& bk = t.buckets[z];
                if (bk.hash == ~0ULL) break;
                if (bk.hash != h) continue;
                const size_t idx = bk.index;
                if (cf.type == CT_COUNTER || cf.type == CT_FREQ) {
                    if ((idx + 1) * 4 <= t.blob.size()) {
                        int32_t c;
                        std::memcpy(&c, t.blob.data() + idx * 4, 4);
                        good = total = c;
                    }
                } else if (cf.type == CT_BORDERS || cf.type == CT_BUCKETS) {
                    const int k = std::max(t.n_classes, 1);
                    if ((idx + 1) * (size_t)k * 4 <= t.blob.size()) {
                        const uint8_t* row = t.blob.data() + idx * (size_t)k * 4;
                        for (int c = 0; c < k; ++c) {
                            int32_t v;
                            std::memcpy(&v, row + 4 * c, 4);
                            total += v;
                            if (cf.type == CT_BORDERS ? c > cf.target_border : c == std::min(cf.target_border, k - 1)) good += v;
                        }
                    }
                } else {
                    if ((idx + 1) * 8 <= t.blob.size()) {
                        float sum;
                        int32_t cnt;
                        std::memcpy(&sum, t.blob.data() + idx * 8, 4);
                        std::memcpy(&cnt, t.blob.data() + idx * 8 + 4, 4);
                        good = sum;
                        total = cnt;
                    }
                }
                break;
            }
        }
    }
    double v;
    if (cf.type == CT_COUNTER || cf.type == CT_FREQ) v = (good + cf.prior_num) / ((double)denominator + cf.prior_denom);
    else v = (good + cf.prior_num) / (total + cf.prior_denom);
    return (float)((v + cf.shift) * cf.scale);
}

// raw model values of documents [d0, d0 + cnt), trees [t0, t1): out[doc][dim], scale applied, bias only when t0 == 0
void eval_block(const Model& m, const Input& in, size_t d0, int cnt, size_t t0, size_t t1, double* out,
                std::vector<uint8_t>& bins, std::vector<uint32_t>& cat_hashes, std::vector<uint32_t>& index) {
    const size_t ncol = m.columns.size();
    bins.assign(ncol * BLOCK, 0);
    const bool cats_used = !m.onehots.empty() || !m.ctrs.empty();
    if (cats_used) {
        cat_hashes.resize(m.cats.size() * BLOCK);
        for (size_t c = 0; c < m.cats.size(); ++c)
            for (int d = 0; d < cnt; ++d) cat_hashes[c * BLOCK + d] = cat_value(in, m.cats[c], d0 + d);
    }
    float vals[BLOCK];
    int last_src = -1;
    Kind last_kind = K_FLOAT;
    for (size_t c = 0; c < ncol; ++c) {
        const Column& col = m.columns[c];
        uint8_t* bc = bins.data() + c * BLOCK;
        if (col.kind == K_ONEHOT) {
            const OneHot& oh = m.onehots[col.src];
            const uint32_t* hv = cat_hashes.data() + (size_t)oh.cat_index * BLOCK;
            for (int j = 0; j < col.count; ++j) {
                const uint32_t want = oh.values[col.first + j];
                for (int d = 0; d < cnt; ++d)
                    if (hv[d] == want) bc[d] = (uint8_t)(j + 1);
            }
            continue;
        }
        const float* borders;
        bool nan_max = false;
        if (col.kind == K_FLOAT) {
            const FloatFeature& f = m.floats[col.src];
            if (!(last_kind == K_FLOAT && last_src == col.src))
                for (int d = 0; d < cnt; ++d) vals[d] = float_value(m, in, f, d0 + d);
            borders = f.borders.data();
            nan_max = f.nan_is_max;
        } else {
            const CtrFeature& cf = m.ctrs[col.src];
            if (!(last_kind == K_CTR && last_src == col.src))
                for (int d = 0; d < cnt; ++d) vals[d] = ctr_value(m, cf, cat_hashes.data(), d);
            borders = cf.borders.data();
        }
        last_kind = col.kind;
        last_src = col.src;
        for (int j = 0; j < col.count; ++j) {
            const float bd = borders[col.first + j];
            for (int d = 0; d < cnt; ++d) bc[d] += (uint8_t)(vals[d] > bd);
        }
        if (col.kind == K_FLOAT)
            for (int d = 0; d < cnt; ++d)
                if (vals[d] != vals[d]) bc[d] = nan_max ? (uint8_t)col.count : (uint8_t)0;
    }

    const int dims = m.dims;
    for (int d = 0; d < cnt; ++d)
        for (int k = 0; k < dims; ++k) out[(size_t)d * dims + k] = 0.0;
    if (m.oblivious) {
        index.resize(BLOCK);
        for (size_t t = t0; t < t1; ++t) {
            const int depth = m.tree_sizes[t];
            const int* sp = m.tree_splits.data() + m.tree_starts[t];
            uint32_t* idx = index.data();
            for (int d = 0; d < BLOCK; ++d) idx[d] = 0;
            for (int lvl = 0; lvl < depth; ++lvl) {
                const BinSplit& bs = m.splits[sp[lvl]];
                const uint8_t* bc = bins.data() + (size_t)bs.column * BLOCK;
                const uint8_t thr = bs.threshold;
                if (bs.equal)
                    for (int d = 0; d < BLOCK; ++d) idx[d] |= (uint32_t)(bc[d] == thr) << lvl;
                else
                    for (int d = 0; d < BLOCK; ++d) idx[d] |= (uint32_t)(bc[d] >= thr) << lvl;
            }
            const double* lv = m.leaf_values.data() + m.tree_leaf_start[t] * dims;
            if (dims == 1)
                for (int d = 0; d < cnt; ++d) out[d] += lv[idx[d]];
            else
                for (int d = 0; d < cnt; ++d)
                    for (int k = 0; k < dims; ++k) out[(size_t)d * dims + k] += lv[(size_t)idx[d] * dims + k];
        }
    } else {
        for (size_t t = t0; t < t1; ++t) {
            const size_t base = m.tree_starts[t], sz = m.tree_sizes[t];
            for (int d = 0; d < cnt; ++d) {
                size_t node = 0;
                for (size_t hops = 0; hops <= sz; ++hops) {
                    if (m.step_left[base + node] == 0 && m.step_right[base + node] == 0) break;      // a leaf
                    const BinSplit& bs = m.splits[m.tree_splits[base + node]];
                    const uint8_t b = bins[(size_t)bs.column * BLOCK + d];
                    const bool right = bs.equal ? b == bs.threshold : b >= bs.threshold;
                    const uint16_t step = right ? m.step_right[base + node] : m.step_left[base + node];
                    if (step == 0 || node + step >= sz) break;
                    node += step;
                }
                const size_t leaf = m.node_to_leaf[base + node];
                if (leaf + dims <= m.leaf_values.size())
                    for (int k = 0; k < dims; ++k) out[(size_t)d * dims + k] += m.leaf_values[leaf + k];
            }
        }
    }
    for (int d = 0; d < cnt; ++d)
        for (int k = 0; k < dims; ++k) {
            double v = out[(size_t)d * dims + k] * m.scale;
            if (t0 == 0) v += m.bias[k];
            out[(size_t)d * dims + k] = v;
        }
}

size_t prediction_dims(const Model& m) {
    if (m.prediction_type == APT_CLASS) return 1;
    return (size_t)m.dims;
}

inline double sigmoid(double x) { return 1.0 / (1.0 + std::exp(-x)); }

// raw[dims] -> res[prediction_dims]
void postprocess(const Model& m, const double* raw, double* res) {
    const int dims = m.dims;
    switch (m.prediction_type) {
        case APT_RAW_FORMULA_VAL:
            for (int k = 0; k < dims; ++k) res[k] = raw[k];
            return;
        case APT_EXPONENT:
            for (int k = 0; k < dims; ++k) res[k] = std::exp(raw[k]);
            return;
        case APT_RMSE_WITH_UNCERTAINTY:
            for (int k = 0; k < dims; ++k) res[k] = raw[k];
            if (dims > 1) res[1] = std::exp(2.0 * raw[1]);
            return;
        case APT_PROBABILITY:
            if (dims == 1) { res[0] = sigmoid(raw[0]); return; }
            {
                double mx = raw[0], sum = 0.0;
                for (int k = 1; k < dims; ++k) mx = std::max(mx, raw[k]);
                for (int k = 0; k < dims; ++k) { res[k] = std::exp(raw[k] - mx); sum += res[k]; }
                for (int k = 0; k < dims; ++k) res[k] /= sum;
            }
            return;
        case APT_MULTI_PROBABILITY:
            for (int k = 0; k < dims; ++k) res[k] = sigmoid(raw[k]);
            return;
        case APT_CLASS:
            if (dims == 1) { res[0] = raw[0] > 0.0 ? 1.0 : 0.0; return; }
            {
                int best = 0;
                for (int k = 1; k < dims; ++k)
                    if (raw[k] > raw[best]) best = k;
                res[0] = best;
            }
            return;
    }
    fail("unknown prediction type");
}

// class_id < 0: all prediction dimensions per document; otherwise that one
void predict(const Model& m, const Input& in, size_t docs, size_t t0, size_t t1, int class_id, double* result,
             size_t result_size) {
    if (m.n_trees() == 0 && m.leaf_values.empty() && m.bias.empty()) fail("no model is loaded");
    check_input(m, in);
    t1 = std::min(t1, m.n_trees());
    if (t0 > t1) fail("treeStart is past treeEnd");
    const size_t pd = class_id < 0 ? prediction_dims(m) : 1;
    if (class_id >= 0 && (size_t)class_id >= prediction_dims(m)) fail("classId is out of range");
    if (result_size < docs * pd) fail("result buffer is too small: need " + std::to_string(docs * pd) + " values");
    if (docs && !result) fail("result pointer is null");
    const long long blocks = (long long)((docs + BLOCK - 1) / BLOCK);
    std::string err;
#pragma omp parallel if (blocks > 8)
    {
        std::vector<uint8_t> bins;
        std::vector<uint32_t> hashes, index;
        std::vector<double> raw((size_t)BLOCK * m.dims), tmp(m.dims);
#pragma omp for schedule(dynamic, 4)
        for (long long b = 0; b < blocks; ++b) {
            try {
                const size_t d0 = (size_t)b * BLOCK;
                const int cnt = (int)std::min<size_t>(BLOCK, docs - d0);
                eval_block(m, in, d0, cnt, t0, t1, raw.data(), bins, hashes, index);
                for (int d = 0; d < cnt; ++d) {
                    if (class_id < 0) {
                        postprocess(m, raw.data() + (size_t)d * m.dims, result + (d0 + d) * pd);
                    } else {
                        postprocess(m, raw.data() + (size_t)d * m.dims, tmp.data());
                        result[d0 + d] = tmp[class_id];
                    }
                }
            } catch (const std::exception& e) {
#pragma omp critical
                err = e.what();
            }
        }
    }
    if (!err.empty()) fail(err);
}

Model& model_of(ModelCalcerHandle* h) {
    if (!h) fail("model handle is null");
    return *static_cast<Model*>(h);
}

template <class F> bool guarded(F&& f) {
    try {
        f();
        return true;
    } catch (const std::exception& e) {
        g_error = e.what();
    } catch (...) {
        g_error = "unknown error";
    }
    return false;
}

bool load_bytes(ModelCalcerHandle* h, const void* data, size_t size) {
    return guarded([&] {
        Model& target = model_of(h);
        if (!data) fail("buffer pointer is null");
        Model fresh;
        parse_model(fresh, static_cast<const uint8_t*>(data), size);
        fresh.prediction_type = target.prediction_type;
        target = std::move(fresh);
    });
}

bool copy_indices(const std::vector<size_t>& v, size_t** indices, size_t* count) {
    return guarded([&] {
        if (!indices || !count) fail("output pointer is null");
        *count = v.size();
        *indices = static_cast<size_t*>(std::malloc(std::max<size_t>(1, v.size()) * sizeof(size_t)));
        if (!*indices) fail("out of memory");
        std::copy(v.begin(), v.end(), *indices);
    });
}

}  // namespace

// ---- the C interface ---------------------------------------------------------------------------------------------------
extern "C" {

ModelCalcerHandle* ModelCalcerCreate(void) {
    try {
        return new Model();
    } catch (...) {
        g_error = "out of memory";
        return nullptr;
    }
}

void ModelCalcerDelete(ModelCalcerHandle* modelHandle) { delete static_cast<Model*>(modelHandle); }

const char* GetErrorString(void) { return g_error.c_str(); }

bool LoadFullModelFromFile(ModelCalcerHandle* modelHandle, const char* filename) {
    std::vector<uint8_t> bytes;
    const bool ok = guarded([&] {
        model_of(modelHandle);
        if (!filename) fail("file name is null");
        FILE* f = std::fopen(filename, "rb");
        if (!f) fail(std::string("cannot open ") + filename);
        uint8_t chunk[1 << 16];
        size_t got;
        while ((got = std::fread(chunk, 1, sizeof(chunk), f)) > 0) bytes.insert(bytes.end(), chunk, chunk + got);
        const bool bad = std::ferror(f) != 0;
        std::fclose(f);
        if (bad) fail(std::string("cannot read ") + filename);
    });
    return ok && load_bytes(modelHandle, bytes.data(), bytes.size());
}

bool LoadFullModelFromBuffer(ModelCalcerHandle* modelHandle, const void* binaryBuffer, size_t binaryBufferSize) {
    return load_bytes(modelHandle, binaryBuffer, binaryBufferSize);
}

bool LoadFullModelZeroCopy(ModelCalcerHandle* modelHandle, const void* binaryBuffer, size_t binaryBufferSize) {
    return load_bytes(modelHandle, binaryBuffer, binaryBufferSize);
}

bool EnableGPUEvaluation(ModelCalcerHandle* modelHandle, int deviceId) {
    (void)deviceId;
    return guarded([&] {
        model_of(modelHandle);
        fail("this library evaluates on the host only");
    });
}

bool GetSupportedEvaluatorTypes(ModelCalcerHandle* modelHandle, enum ECatBoostApiFormulaEvaluatorType** formulaEvaluatorTypes,
                                size_t* formulaEvaluatorTypesCount) {
    return guarded([&] {
        model_of(modelHandle);
        if (!formulaEvaluatorTypes || !formulaEvaluatorTypesCount) fail("output pointer is null");
        auto* arr = static_cast<ECatBoostApiFormulaEvaluatorType*>(std::malloc(sizeof(ECatBoostApiFormulaEvaluatorType)));
        if (!arr) fail("out of memory");
        arr[0] = CBA_FET_CPU;
        *formulaEvaluatorTypes = arr;
        *formulaEvaluatorTypesCount = 1;
    });
}

bool SetPredictionType(ModelCalcerHandle* modelHandle, enum EApiPredictionType predictionType) {
    return guarded([&] {
        if ((int)predictionType < APT_RAW_FORMULA_VAL || (int)predictionType > APT_MULTI_PROBABILITY) fail("unknown prediction type");
        model_of(modelHandle).prediction_type = (int)predictionType;
    });
}

bool SetPredictionTypeString(ModelCalcerHandle* modelHandle, const char* predictionTypeStr) {
    return guarded([&] {
        static const std::pair<const char*, int> names[] = {
            {"RawFormulaVal", APT_RAW_FORMULA_VAL}, {"Exponent", APT_EXPONENT},
            {"RMSEWithUncertainty", APT_RMSE_WITH_UNCERTAINTY}, {"Probability", APT_PROBABILITY},
            {"Class", APT_CLASS}, {"MultiProbability", APT_MULTI_PROBABILITY}};
        if (!predictionTypeStr) fail("prediction type is null");
        for (const auto& nm : names)
            if (std::strcmp(nm.first, predictionTypeStr) == 0) {
                model_of(modelHandle).prediction_type = nm.second;
                return;
            }
        fail(std::string("unknown prediction type '") + predictionTypeStr + "'");
    });
}

static bool run(ModelCalcerHandle* h, Input in, size_t docs, size_t t0, size_t t1, int class_id, double* result, size_t result_size) {
    return guarded([&] { predict(model_of(h), in, docs, t0, t1, class_id, result, result_size); });
}

static Input flat_input(const float** f, size_t fs, bool transposed) {
    Input in;
    in.layout = transposed ? Input::FLAT_TRANSPOSED : Input::FLAT;
    in.floats = f;
    in.floats_size = fs;
    return in;
}

static Input string_input(const float** f, size_t fs, const char*** c, size_t cs) {
    Input in;
    in.layout = Input::SPLIT_STRINGS;
    in.floats = f;
    in.floats_size = fs;
    in.cat_strings = c;
    in.cats_size = cs;
    return in;
}

static Input hashed_input(const float** f, size_t fs, const int** c, size_t cs) {
    Input in;
    in.layout = Input::SPLIT_HASHES;
    in.floats = f;
    in.floats_size = fs;
    in.cat_hashes = c;
    in.cats_size = cs;
    return in;
}

bool CalcModelPredictionFlat(ModelCalcerHandle* h, size_t docCount, const float** floatFeatures, size_t floatFeaturesSize,
                             double* result, size_t resultSize) {
    return run(h, flat_input(floatFeatures, floatFeaturesSize, false), docCount, 0, (size_t)-1, -1, result, resultSize);
}

bool CalcModelPredictionFlatStaged(ModelCalcerHandle* h, size_t docCount, size_t treeStart, size_t treeEnd,
                                   const float** floatFeatures, size_t floatFeaturesSize, double* result, size_t resultSize) {
    return run(h, flat_input(floatFeatures, floatFeaturesSize, false), docCount, treeStart, treeEnd, -1, result, resultSize);
}

bool CalcModelPredictionFlatTransposed(ModelCalcerHandle* h, size_t docCount, const float** floatFeatures,
                                       size_t floatFeaturesSize, double* result, size_t resultSize) {
    return run(h, flat_input(floatFeatures, floatFeaturesSize, true), docCount, 0, (size_t)-1, -1, result, resultSize);
}

bool CalcModelPredictionFlatTransposedStaged(ModelCalcerHandle* h, size_t docCount, size_t treeStart, size_t treeEnd,
                                             const float** floatFeatures, size_t floatFeaturesSize, double* result,
                                             size_t resultSize) {
    return run(h, flat_input(floatFeatures, floatFeaturesSize, true), docCount, treeStart, treeEnd, -1, result, resultSize);
}

bool CalcModelPrediction(ModelCalcerHandle* h, size_t docCount, const float** floatFeatures, size_t floatFeaturesSize,
                         const char*** catFeatures, size_t catFeaturesSize, double* result, size_t resultSize) {
    return run(h, string_input(floatFeatures, floatFeaturesSize, catFeatures, catFeaturesSize), docCount, 0, (size_t)-1, -1,
               result, resultSize);
}

bool CalcModelPredictionStaged(ModelCalcerHandle* h, size_t docCount, size_t treeStart, size_t treeEnd,
                               const float** floatFeatures, size_t floatFeaturesSize, const char*** catFeatures,
                               size_t catFeaturesSize, double* result, size_t resultSize) {
    return run(h, string_input(floatFeatures, floatFeaturesSize, catFeatures, catFeaturesSize), docCount, treeStart, treeEnd,
               -1, result, resultSize);
}

bool CalcModelPredictionSingle(ModelCalcerHandle* h, const float* floatFeatures, size_t floatFeaturesSize,
                               const char** catFeatures, size_t catFeaturesSize, double* result, size_t resultSize) {
    return run(h, string_input(&floatFeatures, floatFeaturesSize, &catFeatures, catFeaturesSize), 1, 0, (size_t)-1, -1, result,
               resultSize);
}

bool CalcModelPredictionSingleStaged(ModelCalcerHandle* h, size_t treeStart, size_t treeEnd, const float* floatFeatures,
                                     size_t floatFeaturesSize, const char** catFeatures, size_t catFeaturesSize,
                                     double* result, size_t resultSize) {
    return run(h, string_input(&floatFeatures, floatFeaturesSize, &catFeatures, catFeaturesSize), 1, treeStart, treeEnd, -1,
               result, resultSize);
}

bool CalcModelPredictionWithHashedCatFeatures(ModelCalcerHandle* h, size_t docCount, const float** floatFeatures,
                                              size_t floatFeaturesSize, const int** catFeatures, size_t catFeaturesSize,
                                              double* result, size_t resultSize) {
    return run(h, hashed_input(floatFeatures, floatFeaturesSize, catFeatures, catFeaturesSize), docCount, 0, (size_t)-1, -1,
               result, resultSize);
}

bool CalcModelPredictionText(ModelCalcerHandle*, size_t, const float**, size_t, const char***, size_t, const char***, size_t,
                             double*, size_t) {
    g_error = "text features are not evaluated by this library";
    return false;
}

bool CalcModelPredictionTextAndEmbeddings(ModelCalcerHandle*, size_t, const float**, size_t, const char***, size_t,
                                          const char***, size_t, const float***, size_t*, size_t, double*, size_t) {
    g_error = "text and embedding features are not evaluated by this library";
    return false;
}

bool PredictSpecificClassFlat(ModelCalcerHandle* h, size_t docCount, const float** floatFeatures, size_t floatFeaturesSize,
                              int classId, double* result, size_t resultSize) {
    return guarded([&] { if (classId < 0) fail("classId is out of range"); }) &&
           run(h, flat_input(floatFeatures, floatFeaturesSize, false), docCount, 0, (size_t)-1, classId, result, resultSize);
}

bool PredictSpecificClass(ModelCalcerHandle* h, size_t docCount, const float** floatFeatures, size_t floatFeaturesSize,
                          const char*** catFeatures, size_t catFeaturesSize, int classId, double* result, size_t resultSize) {
    return guarded([&] { if (classId < 0) fail("classId is out of range"); }) &&
           run(h, string_input(floatFeatures, floatFeaturesSize, catFeatures, catFeaturesSize), docCount, 0, (size_t)-1, classId,
               result, resultSize);
}

bool PredictSpecificClassSingle(ModelCalcerHandle* h, const float* floatFeatures, size_t floatFeaturesSize,
                                const char** catFeatures, size_t catFeaturesSize, int classId, double* result,
                                size_t resultSize) {
    return guarded([&] { if (classId < 0) fail("classId is out of range"); }) &&
           run(h, string_input(&floatFeatures, floatFeaturesSize, &catFeatures, catFeaturesSize), 1, 0, (size_t)-1, classId,
               result, resultSize);
}

bool PredictSpecificClassWithHashedCatFeatures(ModelCalcerHandle* h, size_t docCount, const float** floatFeatures,
                                               size_t floatFeaturesSize, const int** catFeatures, size_t catFeaturesSize,
                                               int classId, double* result, size_t resultSize) {
    return guarded([&] { if (classId < 0) fail("classId is out of range"); }) &&
           run(h, hashed_input(floatFeatures, floatFeaturesSize, catFeatures, catFeaturesSize), docCount, 0, (size_t)-1, classId,
               result, resultSize);
}

int GetStringCatFeatureHash(const char* data, size_t size) {
    return (int)(uint32_t)(city1::hash(data ? data : "", data ? size : 0) & 0xffffffffULL);
}

int GetIntegerCatFeatureHash(long long val) {
    char tmp[24];
    const int len = std::snprintf(tmp, sizeof(tmp), "%lld", val);
    return GetStringCatFeatureHash(tmp, (size_t)len);
}

size_t GetFloatFeaturesCount(ModelCalcerHandle* h) { return h ? static_cast<Model*>(h)->floats.size() : 0; }
size_t GetCatFeaturesCount(ModelCalcerHandle* h) { return h ? static_cast<Model*>(h)->cats.size() : 0; }
size_t GetTextFeaturesCount(ModelCalcerHandle*) { return 0; }
size_t GetEmbeddingFeaturesCount(ModelCalcerHandle*) { return 0; }

bool GetFloatFeatureIndices(ModelCalcerHandle* h, size_t** indices, size_t* count) {
    std::vector<size_t> v;
    return guarded([&] { for (const auto& f : model_of(h).floats) v.push_back((size_t)f.flat); }) && copy_indices(v, indices, count);
}

bool GetCatFeatureIndices(ModelCalcerHandle* h, size_t** indices, size_t* count) {
    std::vector<size_t> v;
    return guarded([&] { for (const auto& c : model_of(h).cats) v.push_back((size_t)c.flat); }) && copy_indices(v, indices, count);
}

bool GetTextFeatureIndices(ModelCalcerHandle* h, size_t** indices, size_t* count) {
    return guarded([&] { model_of(h); }) && copy_indices({}, indices, count);
}

bool GetEmbeddingFeatureIndices(ModelCalcerHandle* h, size_t** indices, size_t* count) {
    return guarded([&] { model_of(h); }) && copy_indices({}, indices, count);
}

size_t GetTreeCount(ModelCalcerHandle* h) { return h ? static_cast<Model*>(h)->n_trees() : 0; }
size_t GetDimensionsCount(ModelCalcerHandle* h) { return h ? (size_t)static_cast<Model*>(h)->dims : 0; }
size_t GetPredictionDimensionsCount(ModelCalcerHandle* h) { return h ? prediction_dims(*static_cast<Model*>(h)) : 0; }

bool CheckModelMetadataHasKey(ModelCalcerHandle* h, const char* keyPtr, size_t keySize) {
    if (!h || !keyPtr) return false;
    const Model& m = *static_cast<Model*>(h);
    return m.info.count(std::string(keyPtr, keySize)) != 0;
}

size_t GetModelInfoValueSize(ModelCalcerHandle* h, const char* keyPtr, size_t keySize) {
    if (!h || !keyPtr) return 0;
    const Model& m = *static_cast<Model*>(h);
    const auto it = m.info.find(std::string(keyPtr, keySize));
    return it == m.info.end() ? 0 : it->second.size();
}

const char* GetModelInfoValue(ModelCalcerHandle* h, const char* keyPtr, size_t keySize) {
    if (!h || !keyPtr) return nullptr;
    const Model& m = *static_cast<Model*>(h);
    const auto it = m.info.find(std::string(keyPtr, keySize));
    return it == m.info.end() ? nullptr : it->second.c_str();
}

bool GetModelUsedFeaturesNames(ModelCalcerHandle* h, char*** featureNames, size_t* featureCount) {
    return guarded([&] {
        const Model& m = model_of(h);
        if (!featureNames || !featureCount) fail("output pointer is null");
        std::vector<std::pair<int, std::string>> used;        // (flat index, name)
        for (const auto& f : m.floats)
            if (!f.borders.empty()) used.emplace_back(f.flat, f.name.empty() ? std::to_string(f.flat) : f.name);
        std::vector<char> cat_used(m.cats.size(), 0);
        for (const auto& oh : m.onehots) cat_used[oh.cat_index] = 1;
        for (const auto& c : m.ctrs)
            for (int p : c.cat_pos) cat_used[p] = 1;
        for (size_t k = 0; k < m.cats.size(); ++k)
            if (cat_used[k]) used.emplace_back(m.cats[k].flat, m.cats[k].name.empty() ? std::to_string(m.cats[k].flat) : m.cats[k].name);
        std::sort(used.begin(), used.end());
        char** arr = static_cast<char**>(std::malloc(std::max<size_t>(1, used.size()) * sizeof(char*)));
        if (!arr) fail("out of memory");
        for (size_t k = 0; k < used.size(); ++k) {
            arr[k] = static_cast<char*>(std::malloc(used[k].second.size() + 1));
            if (!arr[k]) fail("out of memory");
            std::memcpy(arr[k], used[k].second.c_str(), used[k].second.size() + 1);
        }
        *featureNames = arr;
        *featureCount = used.size();
    });
}

}  // extern "C"
