// Replacement for src/compiler/mul/attention.rs of the reference crate: the attention operator of
// the static graph on a B200 through libellm_attn.so (crate ellm-attn-sys).
//
// The struct keeps its fields and `new` / `run` keep their signatures (attention.rs:12-27, 41-76 of
// the snapshot), so `Operator::Attention`, `Tensor::attention` and the executor
// (src/serving/start.rs:69-73) are untouched apart from the one added call `with_geometry`.
// The commented body of `run` (attention.rs:77-155) - the item walk with `assign`, the per-row
// kernel call - is replaced by one call through the C ABI: every worker thread still calls `run`,
// thread 0 launches, the others return and meet the executor's barrier.
//
// NOT COMPILED in the repository that carries this file (no Rust toolchain there).
use std::ptr::{null, null_mut};

use super::super::super::init::send_sync_ptr::{ConstPtr, MutPtr};
use ellm_attn_sys as sys;

/// What the element type must offer the device path: its softmax scale as f32.
pub trait ToF32 {
    fn to_f32(self) -> f32;
}
impl ToF32 for f32 {
    fn to_f32(self) -> f32 {
        self
    }
}
impl ToF32 for f16 {
    fn to_f32(self) -> f32 {
        self as f32
    }
}

#[derive(Clone)]
pub struct Attention<T> {
    q_ptr: ConstPtr<T>,
    k_ptr: ConstPtr<T>,
    v_ptr: ConstPtr<T>,
    output_ptr: MutPtr<T>,
    batch_size: usize,
    attention_head_num: usize,
    kv_head_num: usize,
    head_size: usize,
    kv_strides: Vec<usize>,
    inverse_sqrt_head: T,
    // device side: the library's operator handle (created by with_geometry; the reference leaks its
    // buffers for the life of the process and so does this: no Drop)
    handle: MutPtr<sys::ellm_attn>,
}

impl<T> Attention<T>
where
    T: Copy + ToF32,
{
    /// Same arguments as before.  The pointers must be DEVICE memory holding bf16 (allocate Q, O,
    /// K, V with `ellm_device_alloc` / `ellm_kv_cache_create` where the snapshot uses
    /// `allocate_init`, src/memory/allocator.rs:16-27).  `kv_head_num` is the number of KV heads
    /// (k.shape[1] of the permuted K tensor); a query head h reads KV head h / (heads / kv_heads).
    pub fn new(
        q_ptr: *const T,
        k_ptr: *const T,
        v_ptr: *const T,
        output_ptr: *mut T,
        batch_size: usize,
        attention_head_num: usize,
        kv_head_num: usize,
        head_size: usize,
        kv_strides: Vec<usize>,
        inverse_sqrt_head: T,
    ) -> Self {
        Self {
            q_ptr: ConstPtr { ptr: q_ptr },
            k_ptr: ConstPtr { ptr: k_ptr },
            v_ptr: ConstPtr { ptr: v_ptr },
            output_ptr: MutPtr { ptr: output_ptr },
            batch_size,
            attention_head_num,
            kv_head_num,
            head_size,
            kv_strides,
            inverse_sqrt_head,
            handle: MutPtr { ptr: null_mut() },
        }
    }

    /// What a device needs beyond `new`'s arguments, both known to `Tensor::attention`:
    /// `max_seq` = rows per (sequence, KV head) the K/V buffers hold (k.shape[2] of the permuted K
    /// tensor), `max_interval` = the largest chunk one `run` is given (q.shape[0], the
    /// sequence_chunk_size of src/bin/main.rs:12-15).  Creates the library's handle.
    pub fn with_geometry(mut self, max_seq: usize, max_interval: usize) -> Self {
        let desc = sys::ellm_attn_desc {
            q: self.q_ptr.ptr as *const _,
            k_cache: self.k_ptr.ptr as *mut _,
            v_cache: self.v_ptr.ptr as *mut _,
            out: self.output_ptr.ptr as *mut _,
            lse: null_mut(),
            k_new: null(),   // K/V rows are written into the cache by the projection before (ellm_matmul3)
            v_new: null(),
            max_batch: self.batch_size,
            q_heads: self.attention_head_num,
            kv_heads: self.kv_head_num,
            head_size: self.head_size,
            kv_strides: [self.kv_strides[0], self.kv_strides[1], self.kv_strides[2], self.kv_strides[3]],
            max_seq,
            max_interval,
            scale: self.inverse_sqrt_head.to_f32(),
            dtype: sys::ELLM_DTYPE_BF16,
            device: 0,
            stream: null_mut(),
            r#async: 0,           // run() returns after the stream drained: what the barrier expects
            prefill_kernel: sys::ELLM_PREFILL_AUTO,
        };
        let mut handle: *mut sys::ellm_attn = null_mut();
        let rc = unsafe { sys::ellm_attn_create(&desc, &mut handle) };
        assert_eq!(rc, sys::ELLM_OK, "ellm_attn_create: {}", sys::last_error());
        self.handle = MutPtr { ptr: handle };
        self
    }

    /// Chunk row r of sequence b is the token at position `position_index + r` and attends keys
    /// 0..=position_index + r.  Called by every worker thread; thread 0 launches.
    pub fn run(
        &self,
        position_index: usize,
        position_interval: usize,
        batch_size: usize,
        cpu_num: usize,
        thread_id: usize,
    ) {
        assert!(!self.handle.ptr.is_null(), "Attention::with_geometry was not called");
        let rc = unsafe {
            sys::ellm_attn_run(self.handle.ptr, position_index, position_interval, batch_size, cpu_num, thread_id)
        };
        if rc != sys::ELLM_OK {
            panic!("attention: {}", sys::last_error()); // the crate is panic = "abort"
        }
    }
}

#[cfg(test)]
mod test {
    // The op-level test the snapshot keeps commented out (attention.rs:264-329), live: all-ones
    // Q, K, V with scale 1 - every softmax weight is equal, so every output element is 1.
    // bf16 buffers on the device; needs a B200.
    use super::*;

    fn bf16_ones(n: usize) -> Vec<u16> {
        vec![0x3F80u16; n] // 1.0 in bf16
    }

    unsafe fn to_device(host: &[u16]) -> *mut u16 {
        extern "C" {
            fn cudaMemcpy(dst: *mut std::ffi::c_void, src: *const std::ffi::c_void, n: usize, kind: i32) -> i32;
        }
        let mut p = null_mut();
        assert_eq!(sys::ellm_device_alloc(0, host.len() * 2, &mut p), 0);
        assert_eq!(cudaMemcpy(p, host.as_ptr() as *const _, host.len() * 2, 1), 0);
        p as *mut u16
    }

    #[test]
    fn test_attention_mul() {
        let sequence_chunk_size = 256;
        let sequence_length = 256;
        let batch_size = 16;
        let attention_head_num = 8;
        let kv_head_num = 8;
        let head_size = 128;
        let q_size = sequence_chunk_size * batch_size * attention_head_num * head_size;
        let kv_size = sequence_length * batch_size * kv_head_num * head_size;
        // K/V physically [sequence, batch, kv_head, head_size] as the model code produces them,
        // addressed as [batch, kv_head, sequence, head_size] through the permuted strides
        let k_strides = [batch_size * kv_head_num * head_size, kv_head_num * head_size, head_size, 1];
        let kv_strides2 = vec![k_strides[1], k_strides[2], k_strides[0], k_strides[3]];
        unsafe {
            let q = to_device(&bf16_ones(q_size));
            let k = to_device(&bf16_ones(kv_size));
            let v = to_device(&bf16_ones(kv_size));
            let o = to_device(&vec![0u16; q_size]);
            let operator = Attention::<f32>::new(
                q as *const f32 as *const _,
                k as *const f32 as *const _,
                v as *const f32 as *const _,
                o as *mut f32 as *mut _,
                batch_size,
                attention_head_num,
                kv_head_num,
                head_size,
                kv_strides2,
                1.0,
            )
            .with_geometry(sequence_length, sequence_chunk_size);
            let thread_num: usize = 8;
            for i in 0..thread_num {
                operator.run(0, sequence_chunk_size, batch_size, thread_num, i);
            }
            extern "C" {
                fn cudaMemcpy(dst: *mut std::ffi::c_void, src: *const std::ffi::c_void, n: usize, kind: i32) -> i32;
            }
            let mut got = vec![0u16; q_size];
            assert_eq!(cudaMemcpy(got.as_mut_ptr() as *mut _, o as *const _, q_size * 2, 2), 0);
            assert!(got.iter().all(|&x| x == 0x3F80));
        }
    }
}
