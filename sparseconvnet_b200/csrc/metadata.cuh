// Host-side description of what a scn_metadata object owns on the device: one Grid per
// spatial scale (site hash + row -> key table) and the dense per-filter-offset rulebooks.
#pragma once

#include <atomic>
#include <map>
#include <vector>

#include "common.cuh"

namespace scn {

// Active sites of one spatial scale.
struct Grid {
  KeyLayout layout{};
  long long n_active = 0;
  long long batch_size = 0;
  bool may_have_blank_rows = false;  // input mode 0: rows whose site a later row took over are in no map
  unsigned long long *row_keys = nullptr;  // [n_active] packed key of every feature row
  HashTable table{};                       // key -> row
};

// Dense rulebook.  The reference stores, per filter offset k, a compacted list of
// (input_row, output_row) pairs (Metadata.h:35).  Because every (offset, output row) has at
// most one rule, the same information is kept here as a table
//     nbr[k * n_out + o] = input row feeding output row o through filter offset k, or -1
// which the output-stationary kernels read with coalesced loads and which the builders write
// without compaction, atomics or a host round trip.  `tnbr` is the transposed view
//     tnbr[k * n_in + i] = output row fed by input row i through offset k, or -1
// used by Deconvolution (the reference swaps the two rule columns, CPU/Deconvolution.cpp:35-37);
// it is valid because every (offset, input row) also has at most one rule.
// A rulebook's per-offset rule counts on their way to the host: an asynchronous copy into pinned
// memory and the event recorded behind it.  The multiply-add count the reference's operators
// return needs these totals (CPU/Convolution.cpp:141), and waiting for them where the operator is
// called would leave the GPU idle once per rulebook; a caller that can take the number later is
// handed the ticket instead.  Reference counted: the ticket outlives its rulebook and metadata.
struct CountTicket {
  unsigned long long *host = nullptr;  // [n] pinned
  cudaEvent_t event = nullptr;
  int n = 0, device = 0;
  std::atomic<int> refs{1};
};
void count_ticket_release(CountTicket *t);
int count_ticket_total(CountTicket *t, long long *total);  // waits for the event only

struct Rulebook {
  int n_offsets = 0;  // filter volume K
  long long n_in = 0, n_out = 0;
  int *nbr = nullptr;
  int *tnbr = nullptr;                       // built on first use
  unsigned long long *counts_dev = nullptr;  // [K] rules per offset
  std::vector<long long> counts_host;        // filled on first request (waits for the stream)
  long long total_rules = -1;
  CountTicket *ticket = nullptr;             // counts in flight (rulebook_counts_async)
  bool built = false;
};

int rulebook_counts(Rulebook &rb, cudaStream_t stream);         // fills counts_host/total_rules (waits)
// Starts the copy of the counts if it has not been started; fills counts_host/total_rules without
// waiting if the copy has already landed.  total_rules stays -1 while the copy is in flight.
int rulebook_counts_async(Rulebook &rb, cudaStream_t stream);
int rulebook_transposed(Rulebook &rb, cudaStream_t stream);     // builds tnbr if missing

struct PendingChain;  // metadata.cu: levels of a strided chain whose kernels run on the side stream

}  // namespace scn

struct scn_metadata {
  int dim = 0;
  // Where the tables live and what last touched them: every entry point that takes the object and
  // a stream notes both (scn::md_touch), so that destroying the object can free on the device that
  // owns the memory and, stream-ordered, behind the last work that reads it.
  int device = -1;
  cudaStream_t last_stream = nullptr;
  std::map<std::vector<int64_t>, scn::Grid> grids;             // key: spatial size
  std::map<std::vector<int64_t>, scn::Rulebook> sub_rules;      // key: size | filter
  std::map<std::vector<int64_t>, scn::Rulebook> strided_rules;  // key: in size | filter | stride

  // input-layer rules of the last scn_md_input_layer call: CSR over output rows of the input
  // rows that land on each site, ascending (the order the reference sums them in).
  int input_mode = -1;
  long long input_n_rows = 0, input_n_active = 0;
  int *input_csr_start = nullptr;  // [n_active + 1]
  int *input_csr_rows = nullptr;   // [n_rows]

  scn::CountTicket *last_ticket = nullptr;  // of the last operator that answered "count pending"
  scn::PendingChain *pending = nullptr;     // a strided chain started with scn_md_strided_chain_start, not yet taken over

  int *flags_dev = nullptr;   // device word the kernels OR DeviceFlag bits into
  int *mailbox = nullptr;     // pinned, device-mapped host slot (8 ints) the waited-for integers are posted to
  int *scalars_dev = nullptr; // small device scratch: [0] count, [1] max batch index
};

namespace scn {
// notes the device (first call) and the stream of an operation on `md`; SCN_ERR_BAD_ARG when the
// object is used from another device than the one that holds its tables
int md_touch(scn_metadata *md, cudaStream_t stream);
std::vector<int64_t> make_key(int dim, const int64_t *a, const int64_t *b = nullptr,
                              const int64_t *c = nullptr);
Grid *find_grid(scn_metadata *md, const int64_t *spatial_size);
// finds or builds
int get_submanifold_rulebook(scn_metadata *md, const int64_t *spatial_size,
                             const int64_t *filter_size, cudaStream_t stream, Rulebook **out);
int get_strided_rulebook(scn_metadata *md, const int64_t *input_size, const int64_t *output_size,
                         const int64_t *filter_size, const int64_t *filter_stride,
                         cudaStream_t stream, Rulebook **out);
}  // namespace scn
