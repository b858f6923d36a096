// Symmetric device memory: one same-sized allocation per rank of a single-node job, every
// rank's allocation mapped into every process (NVLink peer loads / stores from kernels), and
// optionally bound to an NVLink multicast object so that one `multimem` store reaches all
// ranks and one `multimem.ld_reduce` sums over them inside the switch (NVLS).
//
// Built on the CUDA virtual-memory-management API: `cuMemCreate` with a POSIX file descriptor
// as the shareable handle, `cuMemMap` of every peer's handle, `cuMulticastCreate` /
// `AddDevice` / `BindMem` for the multicast view.  File descriptors travel between the rank
// processes over Unix sockets (nkipy_b200/parallel/symm.py); this class only produces and
// consumes them.
//
// Life cycle (every rank, in lock step; "barrier" = a host barrier of the job):
//   SymmetricBuffer buf(device, bytes);   fd = buf.export_fd();        -> exchange fds
//   buf.import_peer(r, fd_r) for every other rank r;                   barrier
//   rank 0: mfd = buf.multicast_create(world);                         -> send mfd to all
//   others: buf.multicast_import(mfd);    all: buf.multicast_add_device();   barrier
//   all: buf.multicast_bind();                                         barrier
//   ... kernels use local_ptr() / peer_ptr(r) / multicast_ptr() ...
//   barrier; buf.close();  (unbinds and unmaps before any memory is released)
// A rank must not exit while its memory is still bound to the multicast object and peers may
// still use it: close() in lock step, after a barrier.
//
// Counterpart in the reference: collectives are enabled when a compiled program is loaded
// (spike/src/model.cpp:38-46, nrt_load_collectives); buffers shared between cores are the
// runtime's business there.
#pragma once
#include <cuda.h>

#include <cstdint>
#include <string>
#include <vector>

namespace spike {

class SymmetricBuffer {
 public:
  SymmetricBuffer(int device_ordinal, size_t bytes);
  ~SymmetricBuffer();
  SymmetricBuffer(const SymmetricBuffer&) = delete;
  SymmetricBuffer& operator=(const SymmetricBuffer&) = delete;

  static bool supported(int device_ordinal);             // VMM with POSIX-fd handles
  static bool multicast_supported(int device_ordinal);   // NVLink multicast objects

  size_t size() const { return size_; }                  // rounded up to the granularity
  int device_ordinal() const { return ordinal_; }
  uint64_t local_ptr() const { return static_cast<uint64_t>(local_va_); }

  int export_fd();                                        // a new descriptor per call; the caller closes it
  void import_peer(int rank, int fd);                     // maps the peer's allocation; does not close fd
  uint64_t peer_ptr(int rank) const;                      // 0 when that rank was not imported
  int num_peers() const { return static_cast<int>(peers_.size()); }

  int multicast_create(int num_devices);                  // creator only: returns the descriptor to share
  void multicast_import(int fd);                          // the other ranks
  void multicast_add_device();                            // every rank, before anyone binds
  void multicast_bind();                                  // every rank, after all have added their device
  uint64_t multicast_ptr() const { return static_cast<uint64_t>(mc_va_); }
  bool has_multicast() const { return mc_va_ != 0; }

  void zero();                                            // memset of the local allocation (synchronous)
  void close();
  bool closed() const { return closed_; }

 private:
  struct Peer {
    int rank = -1;
    CUmemGenericAllocationHandle handle = 0;
    CUdeviceptr va = 0;
  };
  void map_handle(CUmemGenericAllocationHandle h, CUdeviceptr* va);
  int ordinal_;
  CUdevice device_ = 0;
  size_t size_ = 0;
  size_t granularity_ = 0;
  CUmemGenericAllocationHandle local_handle_ = 0;
  CUdeviceptr local_va_ = 0;
  std::vector<Peer> peers_;
  CUmemGenericAllocationHandle mc_handle_ = 0;
  CUdeviceptr mc_va_ = 0;
  bool mc_bound_ = false;
  bool closed_ = false;
};

}  // namespace spike
