//! luminal_blum: libblum.so behind luminal's `Compiler` / `Operator` traits.
//!
//! `BlumCompiler<T>` is used where the reference uses `CudaQuantizedCompiler<T>`
//! (crates/luminal_cuda/src/quantized.rs:235-272): it rewrites the nodes directly downstream of the listed
//! Q8_0 weight nodes - a `Matmul<T>` becomes `BlumQuantizedMatmul<T>`, a `CudaGather<T>` becomes
//! `BlumQuantizedGather<T>` - and panics, as the reference does, when a weight feeds anything else or is not
//! input #1.  The operators keep the reference's hand-off (`Operator::process`, src/op.rs:82-90): inputs are
//! `CudaData<T>` / `CudaData<u8>` device buffers, the output is a freshly allocated `CudaSlice<T>` wrapped in a
//! `Tensor`; only the launch is replaced by a call into the C ABI (include/blum.h).
//!
//! Invocation is unchanged:
//! ```ignore
//! cx.compile(
//!     (GenericCompiler::default(),
//!      (luminal_cuda::CudaCompiler::<f16>::default(), luminal_blum::BlumCompiler::<f16>::new(q_weights))),
//!     (&mut input, &mut logits, &mut kv_cache),
//! );
//! ```
//!
//! This crate is source only: it was written without a Rust toolchain and has not been compiled.
#![allow(clippy::missing_safety_doc)]

pub mod ffi;

use std::{
    cell::RefCell,
    ffi::{c_void, CStr},
    marker::PhantomData,
    os::raw::c_int,
    rc::Rc,
    sync::Arc,
};

use cudarc::driver::{CudaContext, CudaSlice, CudaStream, DevicePtr, DevicePtrMut};
use luminal::{
    op::{InputTensor, Operator},
    prelude::*,
};
use luminal_cuda::{binary::CudaGather, matmul::Matmul, CudaData, CudaFloat};
use petgraph::visit::EdgeRef;

/// The element types the C ABI knows (`blum_dtype`).
pub trait BlumFloat: CudaFloat {
    const DTYPE: c_int;
}
impl BlumFloat for f32 {
    const DTYPE: c_int = ffi::BLUM_F32;
}
impl BlumFloat for half::f16 {
    const DTYPE: c_int = ffi::BLUM_F16;
}

/// One `blum_ctx` bound to cudarc's default stream of device 0, so that launches made through the C ABI stay ordered
/// with every untouched luminal op (the reference launches everything on `device.default_stream()`,
/// crates/luminal_cuda/src/quantized.rs:142).
pub struct BlumContext {
    raw: *mut ffi::blum_ctx,
    pub device: Arc<CudaContext>,
    pub stream: Arc<CudaStream>,
}

impl BlumContext {
    pub fn new(device: Arc<CudaContext>) -> Rc<Self> {
        let stream = device.default_stream();
        let mut raw = std::ptr::null_mut();
        let rc = unsafe { ffi::blum_ctx_create(0, &mut raw) };
        assert_eq!(rc, ffi::BLUM_OK, "blum_ctx_create failed ({rc})");
        let rc = unsafe { ffi::blum_ctx_set_stream(raw, stream.cu_stream() as *mut c_void) };
        assert_eq!(rc, ffi::BLUM_OK, "blum_ctx_set_stream failed ({rc})");
        Rc::new(Self { raw, device, stream })
    }

    /// The reference's error convention is `unwrap()`: a failed call panics with the library's message.
    pub fn check(&self, rc: c_int) {
        if rc != ffi::BLUM_OK {
            let msg = unsafe { CStr::from_ptr(ffi::blum_last_error(self.raw)) };
            panic!("libblum error {rc}: {}", msg.to_string_lossy());
        }
    }

    pub fn raw(&self) -> *mut ffi::blum_ctx {
        self.raw
    }
}

impl Drop for BlumContext {
    fn drop(&mut self) {
        unsafe { ffi::blum_ctx_destroy(self.raw) };
    }
}

/// A Q8_0 tensor repacked by the library from the raw GGUF bytes luminal uploads as `CudaData<u8>`
/// (examples/llama/src/loader.rs:156-158).  Built on first use and kept by the operator that owns it.
struct RepackedWeight {
    ctx: Rc<BlumContext>,
    raw: *mut ffi::blum_q8_weight,
    /// device address of the GGUF bytes it was made from: a different buffer means different weights
    source: u64,
}

impl Drop for RepackedWeight {
    fn drop(&mut self) {
        unsafe { ffi::blum_q8_0_weight_free(self.ctx.raw(), self.raw) };
    }
}

fn repack(ctx: &Rc<BlumContext>, cache: &RefCell<Option<RepackedWeight>>, bytes: &CudaSlice<u8>, n: usize, k: usize) -> *mut ffi::blum_q8_weight {
    let (src, _guard) = bytes.device_ptr(&ctx.stream);
    let mut slot = cache.borrow_mut();
    if slot.as_ref().map(|w| w.source) != Some(src) {
        let mut raw = std::ptr::null_mut();
        ctx.check(unsafe { ffi::blum_q8_0_weight_from_gguf_bytes(ctx.raw(), src as *const c_void, n as i64, k as i64, &mut raw) });
        *slot = Some(RepackedWeight { ctx: ctx.clone(), raw, source: src });
    }
    slot.as_ref().unwrap().raw
}

fn dims(st: &ShapeTracker) -> Vec<usize> {
    st.dims().into_iter().map(|d| d.to_usize().unwrap()).collect()
}

/// `y[B*M, N] = x[B*M, K] * W^T`, W a Q8_0 tensor `[N, K]`.  Stands in for `QuantizedMatmul<T>`
/// (crates/luminal_cuda/src/quantized.rs:116-168), which launches one matvec per row of x.
pub struct BlumQuantizedMatmul<T> {
    ctx: Rc<BlumContext>,
    weight: RefCell<Option<RepackedWeight>>,
    _phantom: PhantomData<T>,
}

impl<T> std::fmt::Debug for BlumQuantizedMatmul<T> {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "BlumQuantizedMatmul")
    }
}

impl<T: BlumFloat> BlumQuantizedMatmul<T> {
    pub fn new(ctx: Rc<BlumContext>) -> Self {
        Self { ctx, weight: RefCell::new(None), _phantom: PhantomData }
    }
}

impl<T: BlumFloat> Operator for BlumQuantizedMatmul<T> {
    fn process(&mut self, inp: Vec<(InputTensor, ShapeTracker)>) -> Vec<Tensor> {
        // the weight arrives as a permuted [K, N] view of the [N, K] tensor, as in the reference (quantized.rs:118-121)
        assert!(!inp[1].1.is_contiguous(), "Weight matrix must be column-major");
        let (a_shape, b_shape) = (dims(&inp[0].1), dims(&inp[1].1));
        let (a_dims, b_dims) = (a_shape.len(), b_shape.len());
        let batch = a_shape.iter().take(a_dims - 2).product::<usize>().max(1);
        let (m, k, n) = (a_shape[a_dims - 2], b_shape[b_dims - 2], b_shape[b_dims - 1]);
        let bytes = &inp[1].0.borrowed().downcast_ref::<CudaData<u8>>().unwrap().0;
        let w = repack(&self.ctx, &self.weight, bytes, n, k);
        let x = &inp[0].0.borrowed().downcast_ref::<CudaData<T>>().unwrap().0;
        let mut out = unsafe { self.ctx.stream.alloc::<T>(batch * m * n).unwrap() };
        {
            let (xp, _x) = x.device_ptr(&self.ctx.stream);
            let (yp, _y) = out.device_ptr_mut(&self.ctx.stream);
            self.ctx.check(unsafe {
                ffi::blum_q8_0_matmul(self.ctx.raw(), w, xp as *const c_void, T::DTYPE, yp as *mut c_void, T::DTYPE, (batch * m) as i64)
            });
        }
        vec![Tensor::new(CudaData(out))]
    }
}

/// Embedding rows of a Q8_0 table.  Stands in for `QuantizedGather<T>` (quantized.rs:202-233): token ids arrive as a
/// host `Vec<f32>` and are truncated to integers.
pub struct BlumQuantizedGather<T> {
    ctx: Rc<BlumContext>,
    embed_dim: usize,
    weight: RefCell<Option<RepackedWeight>>,
    _phantom: PhantomData<T>,
}

impl<T> std::fmt::Debug for BlumQuantizedGather<T> {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "BlumQuantizedGather")
    }
}

impl<T: BlumFloat> BlumQuantizedGather<T> {
    pub fn new(ctx: Rc<BlumContext>, embed_dim: usize) -> Self {
        Self { ctx, embed_dim, weight: RefCell::new(None), _phantom: PhantomData }
    }
}

impl<T: BlumFloat> Operator for BlumQuantizedGather<T> {
    fn process(&mut self, inp: Vec<(InputTensor, ShapeTracker)>) -> Vec<Tensor> {
        let ids: Vec<i32> = inp[0].0.borrowed().downcast_ref::<Vec<f32>>().unwrap().iter().map(|v| *v as i32).collect();
        let bytes = &inp[1].0.borrowed().downcast_ref::<CudaData<u8>>().unwrap().0;
        // rows of the table = bytes / (34 bytes per 32 weights * blocks per row)
        let rows = bytes.len() / (self.embed_dim / 32 * 34);
        let w = repack(&self.ctx, &self.weight, bytes, rows, self.embed_dim);
        let ids_dev = self.ctx.stream.memcpy_stod(&ids).unwrap();
        let mut out = unsafe { self.ctx.stream.alloc::<T>(ids.len() * self.embed_dim).unwrap() };
        {
            let (ip, _i) = ids_dev.device_ptr(&self.ctx.stream);
            let (op, _o) = out.device_ptr_mut(&self.ctx.stream);
            self.ctx.check(unsafe { ffi::blum_q8_0_gather(self.ctx.raw(), w, ip as *const i32, ids.len() as i64, op as *mut c_void, T::DTYPE) });
        }
        vec![Tensor::new(CudaData(out))]
    }
}

/// Rewrites the ops directly downstream of the listed Q8_0 weight nodes, exactly where `CudaQuantizedCompiler<T>` does
/// (quantized.rs:244-271).
#[derive(Default, Debug)]
pub struct BlumCompiler<T>(Vec<NodeIndex>, PhantomData<T>);

impl<T> BlumCompiler<T> {
    pub fn new<To: ToIds>(weights: To) -> Self {
        Self(weights.to_ids(), Default::default())
    }
}

impl<T: BlumFloat + Default> Compiler for BlumCompiler<T> {
    type Output = ();
    fn compile<To: ToIdsMut>(&self, graph: &mut Graph, _: To) {
        let ctx = BlumContext::new(CudaContext::new(0).unwrap());
        for weight in downstream(&self.0, graph) {
            for (target, (inp_ind, _, _)) in graph
                .edges_directed(weight, petgraph::Direction::Outgoing)
                .filter_map(|e| e.weight().as_data().map(|i| (e.target(), i)))
                .collect::<Vec<_>>()
            {
                assert_eq!(inp_ind, 1, "Quantized weight {target:?} is the wrong input!");
                let op_node = graph.node_weight_mut(target).unwrap();
                if let Some(gather) = op_node.as_any().downcast_ref::<CudaGather<T>>() {
                    *op_node = Box::new(BlumQuantizedGather::<T>::new(ctx.clone(), gather.embed_dim));
                } else if op_node.as_any().is::<Matmul<T>>() {
                    *op_node = Box::new(BlumQuantizedMatmul::<T>::new(ctx.clone()));
                } else {
                    panic!("Quantized weight {target:?} is an input to a node that isn't a matmul or gather ({op_node:?})");
                }
            }
        }
    }
}
