// The host side of the cache manager and of a step's description, in C++: what runs between two steps on the
// CPU while the GPU waits.
//
// CacheBook keeps what vt-transformer's PageTable and CacheManager keep (vt-transformer/core/vt_pages.hpp:31-134,
// vt-transformer/core/vt_cache.hpp:29-312) in the form this engine uses: a LIFO free list of pages for every group
// of cache slots, a row for every running request with one block-table entry a page, allocation that takes all
// pages of a step or none, pages of a window group given back as soon as the window has passed them, everything
// given back when a request ends.  fill_step packs the description of a step (token ids, positions, sequence of
// every token, offsets, lengths, rows, wanted rows, block-table rows of every group) into the one int32 buffer
// that is copied to the device.  The Python classes in cache/manager.py and engine/batch.py are the interface;
// this file has no CUDA in it and is compiled with the host compiler alone.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

namespace py = pybind11;

namespace {

struct Pool {
    int num_pages = 0;
    std::vector<int> free_list;          // back() is handed out next: 0, 1, 2, ... from a fresh pool
    std::vector<uint8_t> is_free;

    explicit Pool(int n) : num_pages(n), is_free(n, 1) {
        free_list.reserve(n);
        for (int p = n - 1; p >= 0; --p) free_list.push_back(p);
    }
    int free() const { return (int)free_list.size(); }
    int take() {
        const int p = free_list.back();
        free_list.pop_back();
        is_free[p] = 0;
        return p;
    }
    void give(int p) {
        if (p < 0 || p >= num_pages) throw std::invalid_argument("page " + std::to_string(p) + " does not belong to a pool of " + std::to_string(num_pages) + " pages");
        if (is_free[p]) throw std::invalid_argument("page " + std::to_string(p) + " is freed twice");
        is_free[p] = 1;
        free_list.push_back(p);
    }
};

struct Group {
    long long window;                    // keys a token sees, or -1: all
    Pool pool;
    std::vector<int32_t> table;          // [rows, max_pages], -1 where no page is held
    std::vector<int64_t> first_live;     // [rows] first logical page that may still be held
    Group(long long w, int pages, int rows, int max_pages)
        : window(w), pool(pages), table((size_t)rows * max_pages, -1), first_live(rows, 0) {}
};

class CacheBook {
  public:
    CacheBook(int page_size, int max_requests, long long max_seq_len, const std::vector<std::pair<long long, int>>& groups)
        : page_size_(page_size), rows_(max_requests), max_seq_len_(max_seq_len),
          max_pages_((int)((max_seq_len + page_size - 1) / page_size)), lengths_(max_requests, 0), live_(max_requests, 0) {
        if (page_size < 1) throw std::invalid_argument("page_size must be positive");
        for (const auto& g : groups) groups_.emplace_back(g.first, g.second, max_requests, max_pages_);
        for (int r = max_requests - 1; r >= 0; --r) free_rows_.push_back(r);
    }

    int max_pages() const { return max_pages_; }
    int page_size() const { return page_size_; }
    int n_groups() const { return (int)groups_.size(); }
    int free_rows() const { return (int)free_rows_.size(); }

    // -1: every row is taken
    int admit() {
        if (free_rows_.empty()) return -1;
        const int row = free_rows_.back();
        free_rows_.pop_back();
        live_[row] = 1;
        lengths_[row] = 0;
        return row;
    }

    void release(int row) {
        check_row(row);
        for (auto& g : groups_) {
            int32_t* t = &g.table[(size_t)row * max_pages_];
            for (int i = 0; i < max_pages_; ++i)
                if (t[i] >= 0) {
                    g.pool.give(t[i]);
                    t[i] = -1;
                }
            g.first_live[row] = 0;
        }
        lengths_[row] = 0;
        live_[row] = 0;
        free_rows_.push_back(row);
    }

    long long length(int row) const { return lengths_[row]; }

    std::vector<int> free_pages() const {
        std::vector<int> out;
        for (const auto& g : groups_) out.push_back(g.pool.free());
        return out;
    }
    int pool_pages(int group) const { return groups_.at(group).pool.num_pages; }

    std::vector<int> pages_needed(const std::vector<std::pair<int, long long>>& items) const {
        std::vector<int> need(groups_.size(), 0);
        for (const auto& it : items)
            for (size_t gi = 0; gi < groups_.size(); ++gi) need[gi] += missing(groups_[gi], it.first, it.second, nullptr);
        return need;
    }

    // All pages of all items and groups, or none: returns (-1, 0, 0), or (group, needed, free) of the group that is short.
    py::tuple extend(const std::vector<std::pair<int, long long>>& items) {
        for (const auto& it : items) {
            check_row(it.first);
            if (it.second > max_seq_len_)
                throw std::invalid_argument("row " + std::to_string(it.first) + ": length " + std::to_string(it.second) + " is above max_seq_len " + std::to_string(max_seq_len_));
            if (it.second < lengths_[it.first])
                throw std::invalid_argument("row " + std::to_string(it.first) + ": length " + std::to_string(it.second) + " is below the cached length " + std::to_string(lengths_[it.first]));
        }
        for (size_t gi = 0; gi < groups_.size(); ++gi) {
            int total = 0;
            for (const auto& it : items) total += missing(groups_[gi], it.first, it.second, nullptr);
            if (total > groups_[gi].pool.free()) return py::make_tuple((int)gi, total, groups_[gi].pool.free());
        }
        std::vector<int> where;
        for (auto& g : groups_)
            for (const auto& it : items) {
                where.clear();
                missing(g, it.first, it.second, &where);
                for (int logical : where) g.table[(size_t)it.first * max_pages_ + logical] = g.pool.take();
            }
        return py::make_tuple(-1, 0, 0);
    }

    // A step of `add` tokens for each of `rows`: extend, all or nothing.  Returns (group, needed, free, longest
    // length after the step, shortest); group -1: done.
    py::tuple extend_each(const std::vector<int>& rows, int add) {
        std::vector<std::pair<int, long long>> items;
        items.reserve(rows.size());
        long long longest = 0, shortest = -1;
        for (size_t i = 0; i < rows.size(); ++i) {
            check_row(rows[i]);
            for (size_t j = 0; j < i; ++j)
                if (rows[j] == rows[i]) throw std::invalid_argument("row " + std::to_string(rows[i]) + " appears twice in one step");
            const long long len = lengths_[rows[i]] + add;
            items.emplace_back(rows[i], len);
            if (len > longest) longest = len;
            if (shortest < 0 || len < shortest) shortest = len;
        }
        py::tuple r = extend(items);
        return py::make_tuple(r[0], r[1], r[2], longest, shortest < 0 ? 0 : shortest);
    }

    void commit_each(const std::vector<int>& rows, int add) {
        for (int row : rows) commit(row, lengths_[row] + add);
    }

    void commit(int row, long long new_len) {
        check_row(row);
        lengths_[row] = new_len;
        for (auto& g : groups_) {
            if (g.window < 0) continue;
            const long long lo = first_needed_page(g, new_len);
            const long long first = g.first_live[row];
            if (lo > first) {
                int32_t* t = &g.table[(size_t)row * max_pages_];
                for (long long i = first; i < lo && i < max_pages_; ++i)
                    if (t[i] >= 0) {
                        g.pool.give(t[i]);
                        t[i] = -1;
                    }
                g.first_live[row] = lo;
            }
        }
    }

    // numpy views of the book's own memory (valid as long as the book lives)
    py::array_t<int32_t> table(int group, py::object owner) {
        auto& g = groups_.at(group);
        return py::array_t<int32_t>({(py::ssize_t)rows_, (py::ssize_t)max_pages_}, g.table.data(), owner);
    }
    py::array_t<int64_t> lengths(py::object owner) { return py::array_t<int64_t>({(py::ssize_t)rows_}, lengths_.data(), owner); }

    // "" if all is well: no page lost, none held twice, none both held and free; rows consistent
    std::string check() const {
        for (size_t gi = 0; gi < groups_.size(); ++gi) {
            const auto& g = groups_[gi];
            std::vector<uint8_t> held(g.pool.num_pages, 0);
            int n_held = 0;
            for (int r = 0; r < rows_; ++r)
                for (int i = 0; i < max_pages_; ++i) {
                    const int p = g.table[(size_t)r * max_pages_ + i];
                    if (p < 0) continue;
                    if (p >= g.pool.num_pages) return "group " + std::to_string(gi) + ": a table holds a page the pool does not have";
                    if (!live_[r]) return "group " + std::to_string(gi) + ": free row " + std::to_string(r) + " still holds pages";
                    if (held[p]) return "group " + std::to_string(gi) + ": a page is held twice";
                    if (g.pool.is_free[p]) return "group " + std::to_string(gi) + ": a held page is on the free list";
                    held[p] = 1;
                    ++n_held;
                }
            std::vector<uint8_t> seen(g.pool.num_pages, 0);
            for (int p : g.pool.free_list) {
                if (seen[p]) return "group " + std::to_string(gi) + ": a page is on the free list twice";
                seen[p] = 1;
            }
            if (n_held + g.pool.free() != g.pool.num_pages)
                return "group " + std::to_string(gi) + ": " + std::to_string(g.pool.num_pages - n_held - g.pool.free()) + " pages are lost";
        }
        std::vector<uint8_t> seen(rows_, 0);
        int n_live = 0;
        for (int r : free_rows_) {
            if (seen[r]) return "a row is on the free list twice";
            seen[r] = 1;
        }
        for (int r = 0; r < rows_; ++r) n_live += live_[r];
        if (n_live + (int)free_rows_.size() != rows_) return "a row is lost";
        return "";
    }

    // Packs a step.  `host`: the int32 buffer; offs/sizes: where its arrays lie (token ids, positions, sequence of
    // a token, offsets [n + 1], first positions, lengths after the step, rows, wanted rows, then one block-table
    // array [n, n_pages] a group); T, n, W: tokens, sequences and wanted rows the layout has room for (the rest is
    // padding: tokens of no sequence, sequences without tokens, wanted rows that point at themselves, entries -1).
    // `entries`: (row, token ids) in the order of the step; the first position of an entry is its row's cached
    // length.  Returns (tokens, longest context after the step).
    py::tuple fill_step(py::array_t<int32_t, py::array::c_style> host, int T, int n, int W, int n_pages,
                        const std::vector<long long>& offs, const std::vector<long long>& sizes, const py::list& entries,
                        const std::vector<int>& want_flat) {
        if (offs.size() != 8 + groups_.size() || sizes.size() != offs.size()) throw std::invalid_argument("fill_step: the layout does not fit the groups");
        auto buf = host.mutable_unchecked<1>();
        int32_t* base = buf.mutable_data(0);
        const long long total = host.shape(0);
        for (size_t i = 0; i < offs.size(); ++i)
            if (offs[i] < 0 || offs[i] + sizes[i] > total) throw std::invalid_argument("fill_step: the layout is larger than the buffer");
        int32_t *tok = base + offs[0], *pos = base + offs[1], *tseq = base + offs[2], *cu = base + offs[3], *q_start = base + offs[4],
                *kv_len = base + offs[5], *rows = base + offs[6], *want = base + offs[7];
        const int n_live = (int)entries.size();
        if (n_live > n) throw std::invalid_argument("fill_step: more sequences than the layout has room for");
        int at = 0;
        long long max_kv = 0;
        for (int i = 0; i < n_live; ++i) {
            py::tuple e = entries[i].cast<py::tuple>();
            const int row = e[0].cast<int>();
            check_row(row);
            py::sequence ids = e[1].cast<py::sequence>();
            const int len = (int)py::len(ids);
            if (at + len > T) throw std::invalid_argument("fill_step: more tokens than the layout has room for");
            const long long start = lengths_[row];
            cu[i] = at;
            q_start[i] = (int32_t)start;
            kv_len[i] = (int32_t)(start + len);
            rows[i] = row;
            for (int j = 0; j < len; ++j) {
                tok[at + j] = ids[j].cast<int32_t>();
                pos[at + j] = (int32_t)(start + j);
                tseq[at + j] = i;
            }
            at += len;
            if (start + len > max_kv) max_kv = start + len;
            for (size_t gi = 0; gi < groups_.size(); ++gi) {
                int32_t* bt = base + offs[8 + gi] + (size_t)i * n_pages;
                const int32_t* src = &groups_[gi].table[(size_t)row * max_pages_];
                for (int k = 0; k < n_pages; ++k) bt[k] = k < max_pages_ ? src[k] : -1;
            }
        }
        for (int t = at; t < T; ++t) {
            tok[t] = -1;
            pos[t] = 0;
            tseq[t] = -1;
        }
        for (int i = n_live; i <= n; ++i) cu[i] = at;
        for (int i = n_live; i < n; ++i) {
            q_start[i] = 0;
            kv_len[i] = 0;
            rows[i] = 0;
            for (size_t gi = 0; gi < groups_.size(); ++gi) {
                int32_t* bt = base + offs[8 + gi] + (size_t)i * n_pages;
                for (int k = 0; k < n_pages; ++k) bt[k] = -1;
            }
        }
        const int w = (int)want_flat.size();
        if (w > W) throw std::invalid_argument("fill_step: more wanted rows than the layout has room for");
        for (int i = 0; i < w; ++i) want[i] = want_flat[i];
        for (int i = w; i < W; ++i) want[i] = T - (W - i);          // padding rows want themselves
        return py::make_tuple(at, max_kv);
    }

  private:
    void check_row(int row) const {
        if (row < 0 || row >= rows_ || !live_[row]) throw std::invalid_argument("row " + std::to_string(row) + " holds no request");
    }
    long long first_needed_page(const Group& g, long long length) const {
        if (g.window < 0) return 0;
        const long long first_key = length - g.window + 1;
        return first_key > 0 ? first_key / page_size_ : 0;
    }
    // logical pages below ceil(new_len / page_size) that a later token may read and that are not held
    int missing(const Group& g, int row, long long new_len, std::vector<int>* where) const {
        const long long lo = first_needed_page(g, lengths_[row]);
        long long hi = (new_len + page_size_ - 1) / page_size_;
        if (hi > max_pages_) hi = max_pages_;
        const int32_t* t = &g.table[(size_t)row * max_pages_];
        int n = 0;
        for (long long i = lo; i < hi; ++i)
            if (t[i] < 0) {
                ++n;
                if (where) where->push_back((int)i);
            }
        return n;
    }

    int page_size_, rows_;
    long long max_seq_len_;
    int max_pages_;
    std::vector<Group> groups_;
    std::vector<int64_t> lengths_;
    std::vector<uint8_t> live_;
    std::vector<int> free_rows_;
};


// The scheduler's decision for one step, after vt-transformer's scheduler (vt-transformer/core/vt_scheduler.cpp:
// running requests first, then admission in arrival order under max_running_reqs and max_extend_tokens) with what
// this engine adds: portions of prompts (chunk_size), and pre-emption of the youngest running request when the
// running requests' next tokens need more pages than are free.
//
// running: (row, pending tokens, cached tokens, arrival) of the running requests; waiting: pending tokens of the
// waiting requests in queue order.  The function releases the rows of the requests it pre-empts or gives up on and
// admits rows for the requests it lets in, in `book`; the caller moves its request objects accordingly.
// Returns (plan, preempted, gone_running, gone_waiting, admitted):
//   plan          (index, tokens): index >= 0 a running request, -1 - k the k-th waiting request (now admitted)
//   preempted     indices of running requests sent back to the head of the queue, in the order of pre-emption
//   gone_running  indices of running requests that can never go on (alone and too large for the pool)
//   gone_waiting  indices of waiting requests for which the same holds
//   admitted      (k, row) of the waiting requests let in, in order
py::tuple plan_step(CacheBook& book, const std::vector<std::tuple<int, long long, long long, long long>>& running,
                    const std::vector<long long>& waiting, int max_running, long long max_extend_tokens, long long chunk_size) {
    const int n_groups = book.n_groups(), page_size = book.page_size();
    std::vector<char> alive(running.size(), 1);
    std::vector<int> preempted, gone_running, gone_waiting;
    std::vector<std::pair<int, long long>> plan;
    std::vector<std::pair<int, int>> admitted;
    auto portion = [&](long long pending, long long budget) {
        long long n = pending < budget ? pending : budget;
        if (chunk_size > 0 && pending > 1 && n > chunk_size) n = chunk_size;
        return n;
    };
    long long budget = 0;
    std::vector<int> need, free_now;
    for (;;) {
        // single tokens before prompt portions, each kind in arrival order
        std::vector<int> order;
        for (size_t i = 0; i < running.size(); ++i)
            if (alive[i]) order.push_back((int)i);
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
            const bool pa = std::get<1>(running[a]) > 1, pb = std::get<1>(running[b]) > 1;
            if (pa != pb) return !pa;
            return std::get<3>(running[a]) < std::get<3>(running[b]);
        });
        plan.clear();
        budget = max_extend_tokens;
        std::vector<std::pair<int, long long>> items;
        for (int i : order) {
            const long long n = portion(std::get<1>(running[i]), budget);
            if (n > 0) {
                plan.emplace_back(i, n);
                budget -= n;
                items.emplace_back(std::get<0>(running[i]), std::get<2>(running[i]) + n);
            }
        }
        need = book.pages_needed(items);
        free_now = book.free_pages();
        bool fits = true;
        for (int g = 0; g < n_groups; ++g) fits = fits && need[g] <= free_now[g];
        if (fits) break;
        if (order.size() <= 1) {
            for (int i : order) {             // alone and still too large for the pool: it can never go on
                book.release(std::get<0>(running[i]));
                alive[i] = 0;
                gone_running.push_back(i);
            }
            continue;
        }
        int youngest = order[0];
        for (int i : order)
            if (std::get<3>(running[i]) > std::get<3>(running[youngest])) youngest = i;
        book.release(std::get<0>(running[youngest]));
        alive[youngest] = 0;
        preempted.push_back(youngest);
    }
    std::vector<long long> left(n_groups);
    for (int g = 0; g < n_groups; ++g) left[g] = free_now[g] - need[g];
    int n_running = 0;
    for (char a : alive) n_running += a;
    // admission, first come first served; nobody overtakes the head of the queue
    for (size_t k = 0; k < waiting.size() && budget > 0 && preempted.empty(); ++k) {
        if (n_running >= max_running || book.free_rows() == 0) break;
        long long n = portion(waiting[k], budget);
        long long want = (n + page_size - 1) / page_size;
        const long long reserve = n_running > 0 ? n_running : 0;      // a page of head-room for each running request
        bool short_of = false;
        for (int g = 0; g < n_groups; ++g) short_of = short_of || want + reserve > left[g];
        if (short_of) {
            if (n_running == 0 && plan.empty()) {
                // nothing else holds pages: shrink the portion to what fits, or give up
                long long fit = n;
                if (n_groups > 0) {
                    fit = left[0];
                    for (int g = 1; g < n_groups; ++g) fit = left[g] < fit ? left[g] : fit;
                    fit *= page_size;
                }
                if (fit <= 0) {
                    gone_waiting.push_back((int)k);
                    continue;
                }
                n = n < fit ? n : fit;
                want = (n + page_size - 1) / page_size;
            } else {
                break;
            }
        }
        const int row = book.admit();
        admitted.emplace_back((int)k, row);
        plan.emplace_back(-1 - (int)k, n);
        budget -= n;
        ++n_running;
        for (int g = 0; g < n_groups; ++g) left[g] -= want;
    }
    return py::make_tuple(plan, preempted, gone_running, gone_waiting, admitted);
}

}  // namespace

PYBIND11_MODULE(VTB_HOST_MODULE_NAME, m) {
    m.doc() = "host side of the cache manager and of the description of a step";
    py::class_<Pool>(m, "Pool")
        .def(py::init<int>(), py::arg("num_pages"))
        .def_readonly("num_pages", &Pool::num_pages)
        .def_property_readonly("free", &Pool::free)
        .def("take",
             [](Pool& p, int n) -> py::object {      // n pages, or None (and nothing taken) if fewer are free
                 if (n > p.free()) return py::none();
                 py::list out;
                 for (int i = 0; i < n; ++i) out.append(p.take());
                 return std::move(out);
             })
        .def("give", [](Pool& p, const std::vector<int>& pages) {
            for (int page : pages) p.give(page);
        });
    m.def("plan_step", &plan_step, py::arg("book"), py::arg("running"), py::arg("waiting"), py::arg("max_running"),
          py::arg("max_extend_tokens"), py::arg("chunk_size"));
    py::class_<CacheBook>(m, "CacheBook")
        .def(py::init<int, int, long long, const std::vector<std::pair<long long, int>>&>(), py::arg("page_size"),
             py::arg("max_requests"), py::arg("max_seq_len"), py::arg("groups"))
        .def_property_readonly("max_pages", &CacheBook::max_pages)
        .def_property_readonly("free_rows", &CacheBook::free_rows)
        .def("admit", &CacheBook::admit)
        .def("release", &CacheBook::release)
        .def("length", &CacheBook::length)
        .def("free_pages", &CacheBook::free_pages)
        .def("pool_pages", &CacheBook::pool_pages)
        .def("pages_needed", &CacheBook::pages_needed)
        .def("extend", &CacheBook::extend)
        .def("commit", &CacheBook::commit)
        .def("extend_each", &CacheBook::extend_each)
        .def("commit_each", &CacheBook::commit_each)
        .def("table", [](py::object self, int group) { return self.cast<CacheBook&>().table(group, self); })
        .def("lengths", [](py::object self) { return self.cast<CacheBook&>().lengths(self); })
        .def("check", &CacheBook::check)
        .def("fill_step", &CacheBook::fill_step, py::arg("host").noconvert(), py::arg("T"), py::arg("n"), py::arg("W"),
             py::arg("n_pages"), py::arg("offs"), py::arg("sizes"), py::arg("entries"), py::arg("want_flat"));
}
