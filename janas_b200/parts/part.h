// The interfaces of the parts a layer is put together from, and their registry.
//
// A part is built from a PartSpec (its registered kind and its constants), the
// compute dtype and the device.  It says which tensors it needs below a name
// prefix (tensors), takes them (load) and computes (apply / forward).  No part
// knows which model it is in: sizes and constants arrive as parameters,
// everything about the current step arrives in a StepContext.
//
// Outputs of mixers and feed-forwards are *stacks of partial sums*: float32
// [S, n, hidden] whose sum over S is the part's output (S = 1 unless a matrix
// product was split over its inner dimension).  The block adds them to the
// residual stream in the order 0 .. S-1.
//
// A new mixer, feed-forward, norm, position encoding or block arrangement is a
// class registered under a new name (register_part / register_block); a
// configuration then refers to it by that name in a PartSpec.  Nothing else in
// the library has to change.  Parts can also be registered from outside the
// library through the C interface (parts/foreign.cpp): a callback that answers
// the same questions.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../cache/cache.h"
#include "../config/spec.h"
#include "../csrc/launch.h"
#include "../weights/loader.h"

namespace jb {

enum StepKind {
    PREFILL,   // every sequence starts at its first token
    DECODE,    // every sequence goes on by one token
    EXTEND     // anything else (tokens appended to sequences that have some)
};
const char *step_kind_name(StepKind k);

class Norm;

// What a mixer sees of the cache for the run-order entry it runs as.
struct LayerCache {
    ops::AttnCache kv;                  // this entry's K/V pages and the step's block table
    int kv_heads = 0, head_dim = 0, v_head_dim = 0;
    void *state = nullptr;              // [slots, *state shape], indexed by slot; or null
    StateSpec state_spec;
    // floats from one slot's state to the next's where the state is a part of a longer row
    // per slot (a mixer that is one of a pair); 0: the state's own size
    long long state_stride = 0;
    void *block_state = nullptr;        // the block arrangement's own state, [slots, *shape]; or null
    StateSpec block_state_spec;
    int n_slots = 0;
};

// One step: the rows (tokens) it runs and where each belongs.  Rows are the
// sequences' tokens one sequence after the other.  row_pos, row_seq and seq_slot
// are int32 arrays on the device; the seq_* vectors are on the host and empty in
// a captured decode step (which is replayed with other contents).
struct StepContext {
    StepKind kind = PREFILL;
    DType dtype = BF16;
    Device *dev = nullptr;
    long long n_rows = 0;
    int n_seqs = 0;
    long long hidden = 0;                // width of the residual stream
    const int32_t *row_pos = nullptr;    // position of each row in its sequence
    const int32_t *row_seq = nullptr;    // index of the row's sequence within the step
    const int32_t *seq_slot = nullptr;   // slot of each sequence
    std::vector<int> seq_slots;
    std::vector<long long> seq_pos0;     // tokens each sequence had before the step
    std::vector<long long> seq_len;      // tokens each sequence brings
    std::vector<long long> seq_row0;     // first row of each sequence (n_seqs + 1 values)
    const int32_t *tokens = nullptr;     // the rows' token ids, on the device
    // a table of vectors per token beside the embedding (ModelSpec::token_table_name), for
    // blocks that give every layer an input of the token's own; null: the model has none
    const DevTensor *token_table = nullptr;
    long long max_pos = 0;               // the largest position of any row (a bound, in a captured step)
    bool captured = false;               // the launches are being recorded into a graph
    // For finding the first layer that goes wrong: when set, the model copies the
    // residual stream [n_rows, hidden] to the host after every entry of the run
    // order (what is still to be added is added first), one vector per entry.
    std::vector<std::vector<float>> *trace = nullptr;
    // what a part computed once for all layers of this step (the attention's blocks)
    struct Extra { Buf buf; int n = 0; };
    std::map<std::string, Extra> extras;
    // The next norm of the residual stream, when the block that ran last computed
    // it with its own last step (see Block::next_norm); taken by whoever applies
    // that norm next.
    Buf normed;
    const Norm *normed_by = nullptr;
    // The whole first product of the part that ran last, when it took side rows into
    // it (Part::take_side_rows): their columns start at side_col0.
    Stack side;
    long long side_col0 = 0;
    // The first product of two mixers that read the same input (a pair's sides), run once for both
    // (Mixer::share_first_product says where each side's columns start); null: every mixer runs its own.
    const Stack *shared = nullptr;
};

using TensorMap = std::map<std::string, DevTensor>;

class Part {
public:
    Part(const PartSpec &s, DType dt, Device *d) : spec(s), dtype(dt), dev(d) {}
    virtual ~Part() = default;
    // name -> TensorSpec of every tensor this part reads, below prefix (which ends
    // without a dot; an empty prefix means no prefix); appended to out
    virtual void tensors(const std::string &prefix, TensorList &out) const {}
    // Takes its tensors (on the device, in their resident dtype) out of the map.
    virtual void load(const std::string &prefix, TensorMap &t) {}
    virtual size_t weight_bytes() const { return 0; }
    virtual Json info() const { return Json::object(); }
    // Side rows: a matrix over the part's own input that belongs to someone else (a
    // block's gate).  A part that can takes it into its first product, so that one
    // kernel serves both; its forward() then leaves that whole product in ctx.side
    // and says in ctx.side_col0 where the side rows' columns start.  False (and
    // nothing taken) where the part cannot.  Called after load().
    virtual bool take_side_rows(DevTensor &m) { return false; }

    PartSpec spec;
    DType dtype;
    Device *dev;

    // an empty leaf names the prefix itself (a tensor called as its part is)
    static std::string name(const std::string &prefix, const std::string &leaf) {
        return prefix.empty() ? leaf : leaf.empty() ? prefix : prefix + "." + leaf;
    }
    // the tensor `name` out of the map (it is erased there); Error when it is missing
    static DevTensor take(TensorMap &t, const std::string &name);
};

class Norm : public Part {
public:
    using Part::Part;
    // Normalizes the rows of the float32 residual stream x [n, size].  With delta
    // (a stack of partial sums) x += sum(delta) happens first, in place.  With
    // rows (n_out indices on the device) only those rows are normalized and
    // returned.  The result is [n or n_out, size] in out_dt.
    virtual Buf apply(StepContext &ctx, float *x, long long n, DType out_dt, const Stack *delta,
                      const int32_t *rows, long long n_out) = 0;
    // x += mult * (sum a + sum b) in place (b may be null), then the norm of every row.
    // A norm whose kernel takes the add in front of it does both in one pass; the rest
    // run the add as a launch of its own.
    virtual Buf apply_after_add(StepContext &ctx, float *x, long long n, DType out_dt, const Stack &a,
                                const Stack *b, float mult) {
        ops::add_scaled_(*ctx.dev, x, n, size(), a, b, mult);
        return apply(ctx, x, n, out_dt, nullptr, nullptr, 0);
    }
    virtual long long size() const = 0;
    // A norm that works value by value as tanh(alpha x) w + b says so here and gives
    // its parameters, so that a block can take it into the kernel that ends a
    // sublayer; every other norm answers false.
    virtual bool dynamic_tanh(ops::DytParams *out) const { return false; }
    // A norm that is (v - mean) / sqrt(var + eps) * w + b with float32 parameters gives them
    // here (rms: no mean is taken off), so that a block can take it into the kernel that
    // norms a sublayer's result and adds it to the residual stream; the others answer false.
    virtual bool layer_norm(ops::LnParams *out, bool *rms) const { return false; }
};

class PositionEncoding : public Part {
public:
    using Part::Part;
    // Called once the cache's size is known: positions below n will be asked for.
    virtual void prepare(long long n_positions) {}
    virtual const float *cos() const { return nullptr; }     // [n_positions, rotary_dim / 2] or null
    virtual const float *sin() const { return nullptr; }
    virtual int rotary_dim() const { return 0; }
    // true: angle i turns the neighbours (2i, 2i + 1); false: values i and i + rotary_dim / 2
    virtual bool pairs() const { return false; }
    virtual long long n_positions() const { return 1ll << 62; }
};

class Mixer : public Part {
public:
    using Part::Part;
    // Keys and values per position that the cache should hold (none() for nothing).
    virtual KVSpec kv_spec() const { return KVSpec(); }
    // Fixed-size state per sequence (none() for nothing).
    virtual StateSpec state_spec() const { return StateSpec(); }
    // whether the mixer honours LayerCache::state_stride (it can then be one of a pair)
    virtual bool strided_state() const { return false; }
    // The matrix of the mixer's first product over its input (after load()), or null where it has
    // none to share.  An owner of two mixers over the same input may take both matrices into one
    // and tell each mixer with share_first_product(col0) where its columns start in that product's
    // sums; forward() then finds the sums in ctx.shared and runs no first product of its own.
    virtual DevTensor *first_matrix() { return nullptr; }
    virtual void share_first_product(long long col0) {}
    virtual void prepare(long long n_positions) {}
    // Whether the mixer can run a step of this kind.
    virtual bool supports(StepKind kind) const { return true; }
    // True when forward() reads everything that changes between decode steps
    // (positions, slots, block tables) from the context's device arrays only, so
    // that a captured decode step can be replayed with new contents.
    virtual bool graph_safe() const { return false; }
    // h: [n, hidden] in the compute dtype -> stack [S, n, hidden] float32
    virtual Stack forward(StepContext &ctx, const void *h, LayerCache &cache) = 0;
};

class FeedForward : public Part {
public:
    using Part::Part;
    virtual bool graph_safe() const { return true; }
    virtual Stack forward(StepContext &ctx, const void *h) = 0;
};

// The parts of one layer as they are handed to its arrangement.  feed_forward and
// ffn_norm are null for a layer without a feed-forward; the two post norms (on a
// sublayer's result, before it joins the residual stream) are null where the
// layer's spec names none.
struct BlockParts {
    std::unique_ptr<Mixer> mixer;
    std::unique_ptr<FeedForward> feed_forward;
    std::unique_ptr<Norm> mixer_norm, ffn_norm, post_mixer_norm, post_ffn_norm;
};

// The arrangement of one layer's parts around the residual stream.  An
// arrangement may own tensors itself (gates on the residual branches), named below
// the layer's prefix like a part's.
class Block {
public:
    explicit Block(BlockParts p)
        : mixer(std::move(p.mixer)), feed_forward(std::move(p.feed_forward)),
          mixer_norm(std::move(p.mixer_norm)), ffn_norm(std::move(p.ffn_norm)),
          post_mixer_norm(std::move(p.post_mixer_norm)), post_ffn_norm(std::move(p.post_ffn_norm)) {}
    virtual ~Block() = default;
    virtual void tensors(const std::string &prefix, TensorList &out) const {}
    virtual void load(const std::string &prefix, TensorMap &t) {}
    virtual size_t weight_bytes() const { return 0; }
    // Fixed-size state per sequence that the arrangement itself keeps (none() for
    // nothing), beside its mixer's; it arrives in LayerCache::block_state.
    virtual StateSpec state_spec() const { return StateSpec(); }
    // as Mixer::supports and Mixer::graph_safe, for what the arrangement itself does
    virtual bool supports(StepKind) const { return true; }
    virtual bool graph_safe() const { return true; }
    // The norm the NEXT thing applies to the residual stream after this layer
    // (the next layer's first norm, or the model's last one), or null; a block may
    // compute it together with its own last step and leave the result in
    // ctx.normed.  Set by the model before each forward.
    const Norm *next_norm = nullptr;
    // x: the float32 residual stream [n, hidden], updated in place; pending: a
    // stack of partial sums not yet added to x (empty for none), replaced by what
    // this layer leaves to be added.
    virtual void forward(StepContext &ctx, float *x, Stack &pending, LayerCache &cache) = 0;

    std::unique_ptr<Mixer> mixer;
    std::unique_ptr<FeedForward> feed_forward;
    std::unique_ptr<Norm> mixer_norm, ffn_norm, post_mixer_norm, post_ffn_norm;
};

// ------------------------------------------------------------------ registry
using PartFactory = std::function<std::unique_ptr<Part>(const PartSpec &, DType, Device *)>;
using BlockFactory = std::function<std::unique_ptr<Block>(BlockParts, const LayerSpec &, DType, Device *)>;

// role: "mixer", "feed_forward", "norm" or "position"
void register_part(const std::string &role, const std::string &kind, PartFactory f);
void register_block(const std::string &kind, BlockFactory f);
std::vector<std::string> registered_parts(const std::string &role);

std::unique_ptr<Part> build_part(const std::string &role, const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<Mixer> build_mixer(const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<FeedForward> build_feed_forward(const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<Norm> build_norm(const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<PositionEncoding> build_position(const PartSpec &spec, DType dt, Device *dev);
// Builds the layer's parts from its spec and hands them to the arrangement it names.
std::unique_ptr<Block> build_block(const LayerSpec &ls, DType dt, Device *dev);

// Several matrices over the same input as one, rows one after the other, so that
// one product serves them all (the reference dispatches q, k, v as one group and
// gate, up as one: src/llm/model_attn.c:255, src/llm/model_ffn.c:349).  If their
// dtypes differ, the widest is taken.  The sources are released as they are copied.
DevTensor fuse_rows(Device &dev, std::vector<DevTensor> &mats);
// The same along the columns: matrices with equally many rows side by side.
DevTensor fuse_cols(Device &dev, std::vector<DevTensor> &mats);

// the built-in kinds (each file registers its own)
void register_builtin_norms();
void register_builtin_positions();
void register_builtin_mixers();
void register_builtin_feed_forwards();
void register_builtin_blocks();
void register_recurrent_mixers();
void register_routed_feed_forwards();
void register_pair_mixers();

}  // namespace jb

// csrc/convert.cu: element type conversions on the device (bfloat16 <-> float32)
extern "C" int jb_convert(const void *src, int src_dt, void *dst, int dst_dt, long long n,
                          cudaStream_t st);
