// Byte-level BPE word merger: applies the merge table in rank order to one pre-tokenised word.
//
// The word arrives as the byte-alphabet string of the Python tokenizer (UTF-8, one code point per original byte).
// Symbols live in a doubly linked list inside a vector; candidate merges sit in a min-heap keyed by (rank, position), and
// stale heap entries are skipped by re-checking the pair they name -- O(n log n) per word instead of the quadratic rescan.
// The reference tokenizer does the same job in C++ (reference: src/v2/utils/Tokenizer.cpp, BPETokenizer::encode).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace {

struct PairHash {
    size_t operator()(const std::pair<int, int>& p) const noexcept {
        return (static_cast<uint64_t>(static_cast<uint32_t>(p.first)) << 32 | static_cast<uint32_t>(p.second)) * 0x9E3779B97F4A7C15ull >> 7;
    }
};

class Merger {
public:
    // tokens: id -> text; merges: (left text, right text) in rank order
    Merger(const std::vector<std::string>& tokens, const std::vector<std::pair<std::string, std::string>>& merges) {
        vocab_.reserve(tokens.size() * 2);
        for (size_t i = 0; i < tokens.size(); ++i) vocab_.emplace(tokens[i], static_cast<int>(i));   // first id wins
        ranks_.reserve(merges.size() * 2);
        for (size_t r = 0; r < merges.size(); ++r) {
            auto a = vocab_.find(merges[r].first), b = vocab_.find(merges[r].second);
            auto ab = vocab_.find(merges[r].first + merges[r].second);
            if (a == vocab_.end() || b == vocab_.end() || ab == vocab_.end()) continue;          // merge outside the vocabulary
            ranks_.emplace(std::make_pair(a->second, b->second), std::make_pair(static_cast<int>(r), ab->second));
        }
    }

    std::vector<int> encode_word(const std::string& word) const {
        // split into code points (each is one symbol of the byte alphabet)
        struct Sym { int id, prev, next; bool alive; };
        std::vector<Sym> syms;
        std::vector<int> out;
        size_t i = 0;
        while (i < word.size()) {
            const unsigned char c = static_cast<unsigned char>(word[i]);
            const size_t len = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : 4;
            auto it = vocab_.find(word.substr(i, len));
            i += len;
            if (it == vocab_.end()) continue;                                                     // not in the vocabulary: dropped
            const int n = static_cast<int>(syms.size());
            syms.push_back({it->second, n - 1, -1, true});
            if (n > 0) syms[n - 1].next = n;
        }
        if (syms.empty()) return out;
        struct Cand { int rank, left, left_id, right_id; };
        auto cmp = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.left > b.left; };
        std::priority_queue<Cand, std::vector<Cand>, decltype(cmp)> heap(cmp);
        auto push = [&](int l) {
            if (l < 0) return;
            const int r = syms[l].next;
            if (r < 0) return;
            auto it = ranks_.find({syms[l].id, syms[r].id});
            if (it != ranks_.end()) heap.push({it->second.first, l, syms[l].id, syms[r].id});
        };
        for (int s = 0; s + 1 < static_cast<int>(syms.size()); ++s) push(s);
        while (!heap.empty()) {
            const Cand c = heap.top();
            heap.pop();
            const Sym& L = syms[c.left];
            if (!L.alive || L.id != c.left_id || L.next < 0 || syms[L.next].id != c.right_id || !syms[L.next].alive) continue;
            const int r = L.next;
            syms[c.left].id = ranks_.at({c.left_id, c.right_id}).second;
            syms[r].alive = false;
            syms[c.left].next = syms[r].next;
            if (syms[r].next >= 0) syms[syms[r].next].prev = c.left;
            push(syms[c.left].prev);
            push(c.left);
        }
        for (int s = 0; s >= 0; s = syms[s].next) out.push_back(syms[s].id);
        return out;
    }

private:
    std::unordered_map<std::string, int> vocab_;
    std::unordered_map<std::pair<int, int>, std::pair<int, int>, PairHash> ranks_;     // (left id, right id) -> (rank, merged id)
};

}  // namespace

PYBIND11_MODULE(llaminar_b200_bpe, m) {
    py::class_<Merger>(m, "Merger")
        .def(py::init<const std::vector<std::string>&, const std::vector<std::pair<std::string, std::string>>&>())
        .def("encode_word", &Merger::encode_word);
}
