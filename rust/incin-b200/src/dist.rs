//! `DistributedContext::from_env()`, meshes, placements, the rendezvous and the reference transport.
//!
//! The environment contract is the launcher's (`RANK`, `WORLD_SIZE`, `LOCAL_RANK`, `MASTER_ADDR`, `MASTER_PORT`, plus
//! `INCIN_RUN_ID` to keep two jobs on one host apart), as in the reference (crates/incin-core/src/dist/context.rs).
//! [`Rendezvous`] is the N-rank TCP control channel of `libincin_host.so` (hello / accepted frames with a run id,
//! abort and shutdown frames, an all-gather of small blobs used to exchange bootstrap data such as IPC handles);
//! [`ReferenceTransport`] gives the collective semantics on host memory, all ranks' buffers in one call, which is
//! what the multi-rank arithmetic is tested against.
use core::ffi::c_void;
use core::fmt;
use std::ffi::CString;

use incin_b200_sys as sys;

#[derive(Debug, Clone, PartialEq, Eq)]
pub enum DistError {
    /// A required variable is missing or does not parse.
    Env(&'static str),
    /// `rank >= world`, or a mesh whose axes do not multiply to the world size.
    Layout(String),
    /// Rendezvous status code of the library (1 timeout, 2 io, 4 world mismatch, 5 bad rank, 6 run id, 7 rejected,
    /// 8 wrong state, 9 aborted by a peer, 11 duplicate rank ...).
    Rendezvous(i32),
    /// Reference-transport status code (1 argument, 2 integer overflow, 3 dtype / op combination).
    Transport(i32),
}

impl fmt::Display for DistError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        match self {
            DistError::Env(name) => write!(f, "environment variable {name} is missing or malformed"),
            DistError::Layout(why) => write!(f, "{why}"),
            DistError::Rendezvous(code) => write!(f, "rendezvous failed with code {code}"),
            DistError::Transport(code) => write!(f, "reference transport failed with code {code}"),
        }
    }
}

impl std::error::Error for DistError {}

/// Who this process is inside the job.
#[derive(Debug, Clone, PartialEq, Eq)]
pub struct DistributedContext {
    pub rank: u32,
    pub world: u32,
    pub local_rank: u32,
    pub master_addr: String,
    pub master_port: u16,
    pub run_id: String,
}

fn env_num(name: &'static str, default: Option<u32>) -> Result<u32, DistError> {
    match std::env::var(name) {
        Ok(v) => v.trim().parse::<u32>().map_err(|_| DistError::Env(name)),
        Err(_) => default.ok_or(DistError::Env(name)),
    }
}

impl DistributedContext {
    /// Read the launcher's variables.  A process started without them is a world of one.
    pub fn from_env() -> Result<Self, DistError> {
        let world = env_num("WORLD_SIZE", Some(1))?;
        let rank = env_num("RANK", Some(0))?;
        let local_rank = env_num("LOCAL_RANK", Some(rank))?;
        if world == 0 || rank >= world {
            return Err(DistError::Layout(format!("rank {rank} is not inside a world of {world}")));
        }
        let master_addr = std::env::var("MASTER_ADDR").unwrap_or_else(|_| "127.0.0.1".to_string());
        let master_port = env_num("MASTER_PORT", Some(29500))?;
        if master_port > u16::MAX as u32 {
            return Err(DistError::Env("MASTER_PORT"));
        }
        let run_id = std::env::var("INCIN_RUN_ID").unwrap_or_else(|_| "incin".to_string());
        Ok(DistributedContext { rank, world, local_rank, master_addr, master_port: master_port as u16, run_id })
    }

    pub fn is_distributed(&self) -> bool {
        self.world > 1
    }

    /// Join the job's control channel (rank 0 listens, the others connect and are checked against world size and
    /// run id).  `port_offset` keeps the channel off the port the tensor library's own store uses.
    pub fn connect(&self, port_offset: u16, timeout_ms: i32) -> Result<Rendezvous, DistError> {
        let addr = format!("{}:{}", self.master_addr, self.master_port as u32 + port_offset as u32);
        let c_addr = CString::new(addr).map_err(|_| DistError::Env("MASTER_ADDR"))?;
        let c_run = CString::new(self.run_id.clone()).map_err(|_| DistError::Env("INCIN_RUN_ID"))?;
        let mut handle: i64 = 0;
        // SAFETY: both strings are NUL-terminated and outlive the call; `handle` is a valid out pointer.
        let rc = unsafe {
            sys::incin_rdv_connect(self.rank as i32, self.world as i32, c_addr.as_ptr(), c_run.as_ptr(),
                                   self.local_rank as i64, timeout_ms, &mut handle)
        };
        if rc != 0 {
            return Err(DistError::Rendezvous(rc));
        }
        Ok(Rendezvous { handle, world: self.world })
    }
}

/// State of the control channel.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum ChannelState {
    Active,
    ShuttingDown,
    ShutdownDone,
    Failed,
}

/// An open control channel; destroyed on drop.
#[derive(Debug)]
pub struct Rendezvous {
    handle: i64,
    world: u32,
}

impl Rendezvous {
    pub fn state(&self) -> ChannelState {
        // SAFETY: the handle stays valid until drop.
        match unsafe { sys::incin_rdv_state(self.handle) } {
            0 => ChannelState::Active,
            1 => ChannelState::ShuttingDown,
            2 => ChannelState::ShutdownDone,
            _ => ChannelState::Failed,
        }
    }

    /// Error unless the channel is still active (checked before every collective launch: fail-stop).
    pub fn ensure_active(&self) -> Result<(), DistError> {
        // SAFETY: as above.
        match unsafe { sys::incin_rdv_ensure_active(self.handle) } {
            0 => Ok(()),
            rc => Err(DistError::Rendezvous(rc)),
        }
    }

    /// Every rank contributes `mine`; returns the blobs of all ranks in rank order.
    pub fn all_gather(&self, mine: &[u8], timeout_ms: i32) -> Result<Vec<Vec<u8>>, DistError> {
        let n = mine.len();
        let mut all = vec![0u8; n * self.world as usize];
        // SAFETY: `all` holds world * n bytes.
        let rc = unsafe {
            sys::incin_rdv_allgather(self.handle, mine.as_ptr() as *const c_void, n as i32, all.as_mut_ptr() as *mut c_void,
                                     timeout_ms)
        };
        if rc != 0 {
            return Err(DistError::Rendezvous(rc));
        }
        Ok(all.chunks(n.max(1)).map(|c| c.to_vec()).collect())
    }

    /// Device index a peer announced at connect time.
    pub fn peer_device(&self, rank: u32) -> i64 {
        // SAFETY: as above.
        unsafe { sys::incin_rdv_peer_device(self.handle, rank as i32) }
    }

    /// Tell every peer to stop with `code` (they observe it in `ensure_active`).
    pub fn abort(&self, code: i32, timeout_ms: i32) -> Result<(), DistError> {
        // SAFETY: as above.
        match unsafe { sys::incin_rdv_abort(self.handle, code, timeout_ms) } {
            0 => Ok(()),
            rc => Err(DistError::Rendezvous(rc)),
        }
    }

    /// Orderly shutdown handshake.
    pub fn shutdown(&self, timeout_ms: i32) -> Result<(), DistError> {
        // SAFETY: as above.
        match unsafe { sys::incin_rdv_shutdown(self.handle, timeout_ms) } {
            0 => Ok(()),
            rc => Err(DistError::Rendezvous(rc)),
        }
    }
}

impl Drop for Rendezvous {
    fn drop(&mut self) {
        // SAFETY: the handle is destroyed exactly once.
        unsafe { sys::incin_rdv_destroy(self.handle) }
    }
}

/// A device mesh with the three axes the planners use.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub struct Mesh {
    pub dp: u32,
    pub tp: u32,
    pub pp: u32,
}

impl Mesh {
    pub fn single() -> Self {
        Mesh { dp: 1, tp: 1, pp: 1 }
    }

    /// Used by `mesh![dp = 2, tp = 4]`; an unknown axis name panics at the call site.
    pub fn with_axis(mut self, axis: &str, n: u32) -> Self {
        match axis {
            "dp" => self.dp = n,
            "tp" => self.tp = n,
            "pp" => self.pp = n,
            other => panic!("unknown mesh axis `{other}` (dp, tp, pp)"),
        }
        self
    }

    pub fn size(&self) -> u32 {
        self.dp * self.tp * self.pp
    }

    /// The mesh must cover the world exactly, with no empty axis.
    pub fn validate(&self, world: u32) -> Result<(), DistError> {
        if self.dp == 0 || self.tp == 0 || self.pp == 0 {
            return Err(DistError::Layout("a mesh axis of extent 0".to_string()));
        }
        if self.size() != world {
            return Err(DistError::Layout(format!("mesh {}x{}x{} has {} devices, the world has {}", self.dp, self.tp,
                                                 self.pp, self.size(), world)));
        }
        Ok(())
    }

    /// `(dp, pp, tp)` coordinates of a rank; tensor-parallel ranks are adjacent (they share the most traffic).
    pub fn coordinates(&self, rank: u32) -> (u32, u32, u32) {
        let tp = rank % self.tp;
        let pp = (rank / self.tp) % self.pp;
        let dp = rank / (self.tp * self.pp);
        (dp, pp, tp)
    }
}

/// How a tensor is laid out over a mesh axis.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Placement {
    Replicated,
    /// Split along this tensor axis.
    Sharded(usize),
    /// Every rank holds a partial sum.
    PartialSum,
    /// Every rank holds a partial mean.
    PartialMean,
}

impl Placement {
    /// The collective that turns `self` into `to`, if the transition is legal.
    pub fn transition(self, to: Placement) -> Option<&'static str> {
        match (self, to) {
            (a, b) if a == b => Some("none"),
            (Placement::Sharded(_), Placement::Replicated) => Some("all_gather"),
            (Placement::PartialSum, Placement::Replicated) => Some("all_reduce(sum)"),
            (Placement::PartialMean, Placement::Replicated) => Some("all_reduce(mean)"),
            (Placement::PartialSum, Placement::Sharded(_)) => Some("reduce_scatter(sum)"),
            (Placement::Replicated, Placement::Sharded(_)) => Some("slice"),
            (Placement::Sharded(a), Placement::Sharded(b)) if a != b => Some("all_to_all"),
            _ => None,
        }
    }
}

#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum ReduceOp {
    Sum = 0,
    Mean = 1,
    Max = 2,
    Min = 3,
    Prod = 4,
}

/// Collective semantics on host memory: every call takes the buffers of ALL ranks and returns all ranks' results.
#[derive(Debug, Clone, Copy, Default)]
pub struct ReferenceTransport;

const DTYPE_F32: i32 = 0;

fn run_f32(inputs: &[Vec<f32>], out_len: usize,
           f: impl FnOnce(*const *const c_void, *const *mut c_void, i32, i64) -> i32) -> Result<Vec<Vec<f32>>, DistError> {
    let world = inputs.len();
    if world == 0 || inputs.iter().any(|v| v.len() != inputs[0].len()) {
        return Err(DistError::Transport(1));
    }
    let mut outputs: Vec<Vec<f32>> = (0..world).map(|_| vec![0.0f32; out_len]).collect();
    let in_ptrs: Vec<*const c_void> = inputs.iter().map(|v| v.as_ptr() as *const c_void).collect();
    let out_ptrs: Vec<*mut c_void> = outputs.iter_mut().map(|v| v.as_mut_ptr() as *mut c_void).collect();
    let rc = f(in_ptrs.as_ptr(), out_ptrs.as_ptr(), world as i32, inputs[0].len() as i64);
    if rc != 0 {
        return Err(DistError::Transport(rc));
    }
    Ok(outputs)
}

impl ReferenceTransport {
    /// Every rank ends with the reduction of all inputs.
    pub fn all_reduce(&self, inputs: &[Vec<f32>], op: ReduceOp) -> Result<Vec<Vec<f32>>, DistError> {
        let n = inputs.first().map_or(0, |v| v.len());
        // SAFETY: pointer tables and buffers are sized by `run_f32`.
        run_f32(inputs, n, |i, o, w, len| unsafe { sys::incin_ref_all_reduce(i, o, w, len, DTYPE_F32, op as i32) })
    }

    /// Every rank ends with the concatenation of all inputs in rank order.
    pub fn all_gather(&self, inputs: &[Vec<f32>]) -> Result<Vec<Vec<f32>>, DistError> {
        let n = inputs.first().map_or(0, |v| v.len());
        // SAFETY: as above; outputs hold world * n elements.
        run_f32(inputs, n * inputs.len(), |i, o, w, len| unsafe { sys::incin_ref_all_gather(i, o, w, len, DTYPE_F32) })
    }

    /// Rank r ends with slice r of the reduction (`n` must be divisible by the world size).
    pub fn reduce_scatter(&self, inputs: &[Vec<f32>], op: ReduceOp) -> Result<Vec<Vec<f32>>, DistError> {
        let n = inputs.first().map_or(0, |v| v.len());
        if inputs.is_empty() || n % inputs.len() != 0 {
            return Err(DistError::Transport(1));
        }
        // SAFETY: as above; outputs hold n / world elements.
        run_f32(inputs, n / inputs.len(), |i, o, w, len| unsafe {
            sys::incin_ref_reduce_scatter(i, o, w, len, DTYPE_F32, op as i32)
        })
    }

    /// Rank r sends chunk c of its input to rank c.
    pub fn all_to_all(&self, inputs: &[Vec<f32>]) -> Result<Vec<Vec<f32>>, DistError> {
        let n = inputs.first().map_or(0, |v| v.len());
        if inputs.is_empty() || n % inputs.len() != 0 {
            return Err(DistError::Transport(1));
        }
        // SAFETY: as above; outputs hold n elements.
        run_f32(inputs, n, |i, o, w, len| unsafe { sys::incin_ref_all_to_all(i, o, w, len, DTYPE_F32) })
    }
}
