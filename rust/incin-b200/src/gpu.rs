//! Safe front end over the sm_100a kernel library (`libincin_sm100.so`).
//!
//! The kernels take raw device pointers and a CUDA stream, so this crate is allocator-agnostic: a [`DevicePtr`] is
//! whatever the caller's CUDA binding hands out (cudarc, cust, a raw `cudaMalloc`), and the caller keeps ownership.
//! What the wrappers add is the part that can be checked on the host: shapes, leading dimensions, TMA alignment and
//! the mapping from a `Result` to the library's status codes.
use core::ffi::c_void;
use incin_b200_sys as sys;

/// Status codes of the C ABI (`INCIN_OK` = 0).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Error {
    Argument,
    Misaligned,
    Driver,
    TensorMap,
    Launch,
    Unsupported,
    TooLarge,
    Peer,
    Other(i32),
}

fn check(rc: i32) -> Result<(), Error> {
    match rc {
        0 => Ok(()),
        1 => Err(Error::Argument),
        2 => Err(Error::Misaligned),
        3 => Err(Error::Driver),
        4 => Err(Error::TensorMap),
        5 => Err(Error::Launch),
        6 => Err(Error::Unsupported),
        7 => Err(Error::TooLarge),
        8 => Err(Error::Peer),
        x => Err(Error::Other(x)),
    }
}

/// A device address owned by the caller.
#[derive(Debug, Clone, Copy)]
pub struct DevicePtr(pub *mut c_void);

/// A CUDA stream handle (`cudaStream_t`); null is the default stream.
#[derive(Debug, Clone, Copy)]
pub struct Stream(pub *mut c_void);

/// Which way an operand is stored: `K` = rows of the logical matrix are contiguous along the reduction axis.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Major {
    K,
    Mn,
}

/// Activation fused into the GEMM epilogue.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Act {
    None = 0,
    Gelu = 1,
    Silu = 2,
    GeluGrad = 3,
    SiluGrad = 4,
}

/// `C = epilogue(alpha * A @ B^T)` in bf16 with fp32 accumulation on the tcgen05 tensor cores.
pub struct Gemm {
    desc: sys::incin_gemm_desc,
}

impl Gemm {
    /// `a`: `[m, k]`, `b`: `[n, k]` (both K-major, dense), `c`: `[m, n]` bf16.
    pub fn new(a: DevicePtr, b: DevicePtr, c: DevicePtr, m: i32, n: i32, k: i32) -> Self {
        // SAFETY: the descriptor is plain data; all-zero is its documented default.
        let mut d: sys::incin_gemm_desc = unsafe { core::mem::zeroed() };
        d.A = a.0;
        d.B = b.0;
        d.C = c.0;
        d.M = m;
        d.N = n;
        d.K = k;
        d.lda = k as i64;
        d.ldb = k as i64;
        d.ldc = n as i64;
        d.alpha = 1.0;
        d.splits = 1;
        Gemm { desc: d }
    }

    pub fn a_major(mut self, major: Major, lda: i64) -> Self {
        self.desc.a_mn_major = (major == Major::Mn) as i32;
        self.desc.lda = lda;
        self
    }

    pub fn b_major(mut self, major: Major, ldb: i64) -> Self {
        self.desc.b_mn_major = (major == Major::Mn) as i32;
        self.desc.ldb = ldb;
        self
    }

    pub fn bias(mut self, bias: DevicePtr) -> Self {
        self.desc.bias = bias.0;
        self
    }

    pub fn residual(mut self, residual: DevicePtr) -> Self {
        self.desc.residual = residual.0;
        self
    }

    pub fn activation(mut self, act: Act, pre_activation: Option<DevicePtr>) -> Self {
        self.desc.act = act as i32;
        self.desc.aux = pre_activation.map_or(core::ptr::null_mut(), |p| p.0);
        self
    }

    /// fp32 output that is accumulated into (weight gradients); `splits = 0` lets the library pick the split-K factor.
    pub fn accumulate_f32(mut self, splits: i32) -> Self {
        self.desc.out_fp32 = 1;
        self.desc.accumulate = 1;
        self.desc.splits = splits;
        self
    }

    /// Host-side checks the kernel would otherwise reject at launch: TMA moves 16-byte units.
    pub fn validate(&self) -> Result<(), Error> {
        let d = &self.desc;
        if d.M <= 0 || d.N <= 0 || d.K <= 0 {
            return Err(Error::Argument);
        }
        if d.lda % 8 != 0 || d.ldb % 8 != 0 || (d.A as usize) % 16 != 0 || (d.B as usize) % 16 != 0 {
            return Err(Error::Misaligned);
        }
        Ok(())
    }

    pub fn launch(&self, stream: Stream) -> Result<(), Error> {
        self.validate()?;
        // SAFETY: pointers are device addresses supplied by the caller, who guarantees their extents.
        check(unsafe { sys::incin_gemm_bf16(&self.desc, stream.0) })
    }
}

/// RMSNorm forward over `rows x c` bf16; `rstd` (fp32 `[rows]`) is kept for the backward pass.
pub fn rmsnorm_fwd(x: DevicePtr, gamma: DevicePtr, y: DevicePtr, rstd: DevicePtr, rows: i64, c: i32, eps: f32,
                   stream: Stream) -> Result<(), Error> {
    // SAFETY: see `Gemm::launch`.
    check(unsafe { sys::incin_rmsnorm_fwd(x.0, gamma.0, y.0, rstd.0 as *mut f32, rows, c, eps, stream.0) })
}

/// Number of SMs of the current device as the kernel library sees it (148 on a B200).
pub fn num_sms() -> i32 {
    // SAFETY: no arguments, no side effects.
    unsafe { sys::incin_sm100_num_sms() }
}
