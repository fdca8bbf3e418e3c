//! GpuStream / GpuGraph (crates/tl_backend/src/stream.rs:12-31, graph.rs:22-31) over the library's one stream.
use tl_backend::graph::GpuGraph;
use tl_backend::stream::GpuStream;

use crate::ffi;

pub struct B200Stream;

pub struct B200Graph(*mut ffi::TlbGraph);
// the handle is only replayed / destroyed through the library, which orders everything on its own stream
unsafe impl Send for B200Graph {}
unsafe impl Sync for B200Graph {}

impl GpuStream for B200Stream {
    type Graph = B200Graph;

    fn synchronize(&mut self) {
        unsafe { ffi::tlb_sync() };
    }
    /// Work is stream-ordered and results are read through calls that synchronise themselves, so nothing is ever pending
    /// from the caller's point of view (the reference's CUDA stream syncs after every launch instead,
    /// crates/tl_cuda/src/stream.rs:63-73).
    fn needs_sync(&self) -> bool {
        false
    }
    fn begin_capture(&mut self) {
        unsafe { ffi::tlb_stream_begin_capture() };
    }
    fn end_capture(&mut self) -> B200Graph {
        let mut g: *mut ffi::TlbGraph = std::ptr::null_mut();
        unsafe { ffi::tlb_stream_end_capture(&mut g) };
        B200Graph(g)
    }
    fn is_capturing(&self) -> bool {
        unsafe { ffi::tlb_stream_is_capturing() != 0 }
    }
}

impl GpuGraph for B200Graph {
    fn replay(&self) {
        if !self.0.is_null() {
            unsafe { ffi::tlb_graph_replay(self.0) };
        }
    }
    fn node_count(&self) -> usize {
        unsafe { ffi::tlb_graph_node_count(self.0) }.max(0) as usize
    }
}

impl Drop for B200Graph {
    fn drop(&mut self) {
        unsafe { ffi::tlb_graph_destroy(self.0) };
    }
}
