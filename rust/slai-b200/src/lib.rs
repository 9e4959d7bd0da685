//! Safe wrappers over the C ABI of `libslai_b200.so` (`include/slai_b200.h`).
//!
//! The types keep the names and the argument meaning of the reference crate (`crates/slai/src`), so that code written
//! against `GemvQuant::launch`, `RmsNorm::launch`, ... changes its backend type and nothing else.  Each item cites the
//! reference interface it stands for.
use slai_b200_sys as sys;
pub use slai_b200_sys::B200Error;
use std::marker::PhantomData;
use std::os::raw::c_void;
use std::ptr;

pub mod models;
pub mod ops;

/// One CUDA context + stream on one GPU: what `B: Backend` is to the reference (`LlmOps::new`,
/// crates/slai/src/context.rs:47-66).  Not `Sync`: one host thread drives a context at a time; several contexts (one
/// per GPU) are independent.
pub struct B200 {
    pub(crate) h: *mut sys::slai_ctx,
}
unsafe impl Send for B200 {}

impl B200 {
    pub fn new(device: i32) -> Result<Self, B200Error> {
        let mut h = ptr::null_mut();
        let rc = unsafe { sys::slai_ctx_create(device, &mut h) };
        if rc != sys::SLAI_OK {
            return Err(B200Error::Cuda(format!("slai_ctx_create({device}) failed with status {rc}")));
        }
        Ok(B200 { h })
    }
    pub fn device_count() -> i32 {
        unsafe { sys::slai_device_count() }
    }
    pub(crate) fn check(&self, rc: i32) -> Result<(), B200Error> {
        unsafe { sys::check(rc, self.h) }
    }
    /// Blocks until everything queued so far has run; reports a device-side wait that ran out as `Timeout`.
    pub fn synchronize(&self) -> Result<(), B200Error> {
        self.check(unsafe { sys::slai_ctx_sync(self.h) })
    }
    /// `LlmContext::begin_submission` (context.rs:79-88).
    pub fn begin_submission(&self) -> B200Pass<'_> {
        B200Pass { backend: self }
    }
    /// Uninitialised device vector of `n` elements.
    pub fn alloc<T: Copy>(&self, n: usize) -> Result<DeviceVec<'_, T>, B200Error> {
        let mut p: *mut c_void = ptr::null_mut();
        self.check(unsafe { sys::slai_malloc(self.h, n * std::mem::size_of::<T>(), &mut p) })?;
        Ok(DeviceVec { backend: self, ptr: p as *mut T, len: n })
    }
    pub fn zeros<T: Copy>(&self, n: usize) -> Result<DeviceVec<'_, T>, B200Error> {
        let v = self.alloc::<T>(n)?;
        self.check(unsafe { sys::slai_memset(self.h, v.ptr as *mut c_void, 0, n * std::mem::size_of::<T>()) })?;
        Ok(v)
    }
    pub fn vector<T: Copy>(&self, data: &[T]) -> Result<DeviceVec<'_, T>, B200Error> {
        let v = self.alloc::<T>(data.len())?;
        self.check(unsafe { sys::slai_write_buffer(self.h, v.ptr as *mut c_void, data.as_ptr() as *const c_void, std::mem::size_of_val(data)) })?;
        Ok(v)
    }
    /// Sets how many polls a bounded device-side wait takes before it gives up (default about a second).
    pub fn set_wait_limit(&self, rounds: u32) -> Result<(), B200Error> {
        self.check(unsafe { sys::slai_ctx_set_wait_limit(self.h, rounds) })
    }
}
impl Drop for B200 {
    fn drop(&mut self) {
        unsafe { sys::slai_ctx_destroy(self.h) };
    }
}

/// Stands where `B::Pass` stands in the reference's `launch` signatures.  Operators queue their kernels on the
/// context's stream as they are called; `submit` is the point after which results may be read.
pub struct B200Pass<'a> {
    pub(crate) backend: &'a B200,
}
impl<'a> B200Pass<'a> {
    /// `LlmContext::submit` (context.rs:90-95).
    pub fn submit(self) -> Result<(), B200Error> {
        self.backend.synchronize()
    }
}

/// Owned device memory of `len` elements (`GpuTensor` / `GpuVector` of the reference).
pub struct DeviceVec<'a, T: Copy> {
    pub(crate) backend: &'a B200,
    pub(crate) ptr: *mut T,
    pub(crate) len: usize,
}
impl<'a, T: Copy> DeviceVec<'a, T> {
    pub fn len(&self) -> usize {
        self.len
    }
    pub fn is_empty(&self) -> bool {
        self.len == 0
    }
    pub fn view(&self) -> View<'_, T> {
        View { ptr: self.ptr, len: self.len, _p: PhantomData }
    }
    pub fn view_mut(&mut self) -> ViewMut<'_, T> {
        ViewMut { ptr: self.ptr, len: self.len, _p: PhantomData }
    }
    /// Elements `[offset, offset + len)` (the reference's `GpuTensorView` of a column, transformer.rs:329-334).
    pub fn slice_mut(&mut self, offset: usize, len: usize) -> ViewMut<'_, T> {
        assert!(offset + len <= self.len);
        ViewMut { ptr: unsafe { self.ptr.add(offset) }, len, _p: PhantomData }
    }
    pub fn slice(&self, offset: usize, len: usize) -> View<'_, T> {
        assert!(offset + len <= self.len);
        View { ptr: unsafe { self.ptr.add(offset) }, len, _p: PhantomData }
    }
    pub fn write(&mut self, data: &[T]) -> Result<(), B200Error> {
        assert!(data.len() <= self.len);
        self.backend.check(unsafe { sys::slai_write_buffer(self.backend.h, self.ptr as *mut c_void, data.as_ptr() as *const c_void, std::mem::size_of_val(data)) })
    }
    /// Blocking read-back (`slow_read_buffer` of the reference's backend).
    pub fn to_vec(&self) -> Result<Vec<T>, B200Error> {
        let mut out = Vec::<T>::with_capacity(self.len);
        self.backend.check(unsafe { sys::slai_read_buffer(self.backend.h, out.as_mut_ptr() as *mut c_void, self.ptr as *const c_void, self.len * std::mem::size_of::<T>()) })?;
        unsafe { out.set_len(self.len) };
        Ok(out)
    }
}
impl<'a, T: Copy> Drop for DeviceVec<'a, T> {
    fn drop(&mut self) {
        unsafe { sys::slai_free(self.backend.h, self.ptr as *mut c_void) };
    }
}

/// Borrowed read-only device range.
#[derive(Copy, Clone)]
pub struct View<'a, T> {
    pub(crate) ptr: *const T,
    pub(crate) len: usize,
    _p: PhantomData<&'a T>,
}
/// Borrowed writable device range.
pub struct ViewMut<'a, T> {
    pub(crate) ptr: *mut T,
    pub(crate) len: usize,
    _p: PhantomData<&'a mut T>,
}
impl<'a, T> View<'a, T> {
    pub fn len(&self) -> usize {
        self.len
    }
}
impl<'a, T> ViewMut<'a, T> {
    pub fn len(&self) -> usize {
        self.len
    }
}
impl<'a, T: Copy> From<&'a DeviceVec<'_, T>> for View<'a, T> {
    fn from(v: &'a DeviceVec<'_, T>) -> Self {
        v.view()
    }
}
impl<'a, T: Copy> From<&'a mut DeviceVec<'_, T>> for ViewMut<'a, T> {
    fn from(v: &'a mut DeviceVec<'_, T>) -> Self {
        v.view_mut()
    }
}

/// GGUF tensor formats (`GgmlType` values the reference uploads, crates/slai/src/gguf.rs:133-194).
#[repr(i32)]
#[derive(Copy, Clone, Debug, PartialEq, Eq)]
pub enum QuantFormat {
    F32 = 0,
    Q4_0 = 2,
    Q4_1 = 3,
    Q5_0 = 6,
    Q5_1 = 7,
    Q8_0 = 8,
    Q4K = 12,
    Q5K = 13,
    Q6K = 14,
    Q8K = 15,
}

/// `GpuQuantMatrix<B>` (crates/slai/src/quantized_matrix.rs:11-22), built like `GgufTensorData::to_gpu_matrix`
/// (gguf.rs:133-194) from the raw blocks of a GGUF tensor, rows in file order.
pub struct GpuQuantMatrix<'a> {
    pub(crate) backend: &'a B200,
    pub(crate) h: *mut sys::slai_qmatrix,
}
impl<'a> GpuQuantMatrix<'a> {
    pub fn from_blocks(backend: &'a B200, fmt: QuantFormat, nrows: usize, ncols: usize, blocks: &[u8]) -> Result<Self, B200Error> {
        let mut h = ptr::null_mut();
        backend.check(unsafe { sys::slai_qmatrix_create(backend.h, fmt as i32, nrows as i64, ncols as i64, blocks.as_ptr() as *const c_void, blocks.len(), &mut h) })?;
        Ok(GpuQuantMatrix { backend, h })
    }
    /// `GpuQuantMatrix::shape` (quantized_matrix.rs:25-38): `[nrows, ncols]` in dequantised elements.
    pub fn shape(&self) -> [usize; 2] {
        let (mut f, mut r, mut c) = (0i32, 0i64, 0i64);
        unsafe { sys::slai_qmatrix_shape(self.h, &mut f, &mut r, &mut c) };
        [r as usize, c as usize]
    }
    /// Every block's `dequantize()` evaluated on the device, row-major (bit-exact with quantization.rs).
    pub fn dequantize(&self) -> Result<Vec<f32>, B200Error> {
        let [r, c] = self.shape();
        let out = self.backend.alloc::<f32>(r * c)?;
        self.backend.check(unsafe { sys::slai_qmatrix_dequantize(self.backend.h, self.h, out.ptr) })?;
        out.to_vec()
    }
}
impl<'a> Drop for GpuQuantMatrix<'a> {
    fn drop(&mut self) {
        unsafe { sys::slai_qmatrix_destroy(self.h) };
    }
}

/// KV-cache element type (the reference keeps f32, transformer.rs:87-106; f16 halves the second-largest byte stream).
#[repr(i32)]
#[derive(Copy, Clone, Debug, PartialEq, Eq)]
pub enum KvDtype {
    F32 = 0,
    F16 = 1,
}
