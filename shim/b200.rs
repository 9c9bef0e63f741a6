//! `hashline/src/gpu/b200.rs` — the binding of `libhl_b200.so` (include/hl_b200.h) behind the prover's accelerator seams.
//!
//! NOT COMPILED IN THIS REPOSITORY: the image this library is built in has no Rust toolchain.  The file is the source a
//! maintainer drops beside `gpu/metal.rs` and `gpu/cuda.rs` (feature `gpu-b200`; `build.rs` adds
//! `cargo:rustc-link-lib=dylib=hl_b200`).  It implements `zkp_core::pcs::{Backend, EncodedStore}`
//! (zkp-core/src/pcs/backend.rs:30-100) and `zkp_core::sumcheck::SumcheckRounds` (zkp-core/src/sumcheck/rounds.rs:22-28) and
//! reports every non-zero status through `super::declined` (gpu/mod.rs:80-94), so that under `HL_GPU_REQUIRED=1` a decline
//! is fatal and otherwise the CPU body runs.  The C prototypes below are checked against the header by
//! tests/c_abi/abi_smoke.c of the library's repository.
use std::ffi::CStr;
use std::os::raw::{c_char, c_int, c_void};
use std::sync::OnceLock;

use zkp_core::field::{Fp, Fp2};
use zkp_core::merkle::Digest;
use zkp_core::ntt::NttTables;
use zkp_core::pcs::{Backend, EncodedStore, PcsParams};
use zkp_core::sumcheck::SumcheckRounds;

#[repr(C)]
pub struct HlCtx {
    _p: [u8; 0],
}
#[repr(C)]
pub struct HlStore {
    _p: [u8; 0],
}
#[repr(C)]
pub struct HlRounds {
    _p: [u8; 0],
}

extern "C" {
    fn hl_b200_init(device: c_int, out: *mut *mut HlCtx) -> c_int;
    fn hl_b200_label(ctx: *mut HlCtx) -> *const c_char;
    fn hl_b200_last_error(ctx: *mut HlCtx) -> *const c_char;
    fn hl_b200_commit(ctx: *mut HlCtx, log_cols: u32, inv_rate: u32, data: *const u64, rows: usize, max_log: u32, key32: *const u8,
                      store: *mut *mut HlStore, leaves32: *mut u8) -> c_int;
    fn hl_b200_commit_zk(ctx: *mut HlCtx, log_cols: u32, inv_rate: u32, data: *const u64, rows: usize, pads: *const u64, q: usize,
                         pows: *const u64, max_log: u32, key32: *const u8, store: *mut *mut HlStore, leaves32: *mut u8) -> c_int;
    fn hl_b200_commit_zk_packed(ctx: *mut HlCtx, log_cols: u32, inv_rate: u32, packed: *const c_void, row_width: *const u8, rows: usize,
                                pads: *const u64, q: usize, pows: *const u64, max_log: u32, key32: *const u8, salts32: *const u8,
                                leaf_key32: *const u8, node_key32: *const u8, store: *mut *mut HlStore, leaves32: *mut u8,
                                levels_out: *mut u8) -> c_int;
    fn hl_b200_verify_opening(ctx: *mut HlCtx, log_cols: u32, inv_rate: u32, q: usize, pows: *const u64, vecs: *const u64, k: usize, cols: *const u64,
                              rows: usize, ncols: usize, idx: *const u64, salts32: *const u8, paths32: *const u8, depth: u32, root32: *const u8,
                              column_key32: *const u8, leaf_key32: *const u8, node_key32: *const u8, rhos: *const u64, verdict: *mut i32,
                              first_bad: *mut i64) -> c_int;
    fn hl_b200_verify_columns(ctx: *mut HlCtx, cols: *const u64, rows: usize, ncols: usize, idx: *const u64, salts32: *const u8,
                              paths32: *const u8, depth: u32, root32: *const u8, column_key32: *const u8, leaf_key32: *const u8,
                              node_key32: *const u8, rhos: *const u64, k: usize, wants: *const u64, vec_store: *const HlStore,
                              verdict: *mut i32, first_bad: *mut i64) -> c_int;
    fn hl_b200_store_fold(s: *mut HlStore, rhos: *const u64, k: usize, with_pads: c_int, out: *mut u64) -> c_int;
    fn hl_b200_store_columns(s: *mut HlStore, idx: *const u64, nidx: usize, out: *mut u64) -> c_int;
    fn hl_b200_store_free(s: *mut HlStore);
    fn hl_b200_rounds_new(ctx: *mut HlCtx, poly: c_int, k: usize, n_vars: u32, degree: u32, tables: *const u64, coefs: *const u64,
                          ncoefs: usize, out: *mut *mut HlRounds) -> c_int;
    fn hl_b200_rounds_new_ir(ctx: *mut HlCtx, k: usize, n_vars: u32, degree: u32, tables: *const u64, words: *const u32, n_words: usize,
                             n_nodes: u32, n_terms: u32, coefs: *const u64, ncoefs: usize, out: *mut *mut HlRounds) -> c_int;
    fn hl_b200_rounds_round(r: *mut HlRounds, j: u32, eval_one: c_int, sums: *mut u64) -> c_int;
    fn hl_b200_rounds_fold(r: *mut HlRounds, challenge: *const u64) -> c_int;
    fn hl_b200_rounds_finals(r: *mut HlRounds, out: *mut u64) -> c_int;
    fn hl_b200_rounds_free(r: *mut HlRounds);
}

/// the process-wide context, made on first use (as the Metal context is, gpu/metal.rs:75-95); 0 = no device
fn ctx() -> *mut HlCtx {
    static CTX: OnceLock<usize> = OnceLock::new();
    *CTX.get_or_init(|| {
        let mut h: *mut HlCtx = std::ptr::null_mut();
        let dev = std::env::var("HL_B200_DEVICE").ok().and_then(|v| v.parse().ok()).unwrap_or(0);
        if unsafe { hl_b200_init(dev, &mut h) } != 0 {
            return 0;
        }
        h as usize
    }) as *mut HlCtx
}

pub fn enabled() -> bool {
    std::env::var("HL_GPU").map(|v| v == "1").unwrap_or(false) && !ctx().is_null()
}

pub fn label() -> String {
    let c = ctx();
    if c.is_null() {
        return "hl_b200: no device".to_string();
    }
    unsafe { CStr::from_ptr(hl_b200_label(c)) }.to_string_lossy().into_owned()
}

fn last_error() -> String {
    let c = ctx();
    if c.is_null() {
        return "no context".to_string();
    }
    unsafe { CStr::from_ptr(hl_b200_last_error(c)) }.to_string_lossy().into_owned()
}

fn status(rc: c_int) -> Result<(), String> {
    if rc == 0 {
        Ok(())
    } else {
        Err(format!("hl_b200 status {rc}: {}", last_error()))
    }
}

/// `Fp` is `#[repr(transparent)]` over `u64` and `Fp2` is two of them in order (field.rs:19-20, 138-141)
fn words(v: &[Fp]) -> *const u64 {
    v.as_ptr() as *const u64
}

pub struct B200Commit {
    h: *mut HlStore,
    rows: usize,
    n: usize,
    q: usize,
}
// the library serialises the calls of a context behind its own lock
unsafe impl Sync for B200Commit {}
unsafe impl Send for B200Commit {}
impl Drop for B200Commit {
    fn drop(&mut self) {
        unsafe { hl_b200_store_free(self.h) }
    }
}

impl B200Commit {
    fn fold(&self, rhos: &[Vec<Fp2>], with_pads: c_int, width: usize) -> Result<Vec<Vec<Fp2>>, String> {
        let k = rhos.len();
        let mut flat: Vec<u64> = Vec::with_capacity(k * self.rows * 2);
        for rho in rhos {
            if rho.len() != self.rows {
                return Err(format!("fold: a weight vector of {} entries for {} rows", rho.len(), self.rows));
            }
            for x in rho {
                flat.push(x.c0.0);
                flat.push(x.c1.0);
            }
        }
        let mut out = vec![0u64; k * width * 2];
        status(unsafe { hl_b200_store_fold(self.h, flat.as_ptr(), k, with_pads, out.as_mut_ptr()) })?;
        Ok((0..k).map(|g| (0..width).map(|j| Fp2 { c0: Fp(out[(g * width + j) * 2]), c1: Fp(out[(g * width + j) * 2 + 1]) }).collect()).collect())
    }
}

impl EncodedStore for B200Commit {
    fn fold_rows(&self, rhos: &[Vec<Fp2>]) -> Result<Vec<Vec<Fp2>>, String> {
        self.fold(rhos, 0, self.n)
    }
    fn columns(&self, idx: &[usize]) -> Result<Vec<Vec<Fp>>, String> {
        let ix: Vec<u64> = idx.iter().map(|&j| j as u64).collect();
        let mut out = vec![Fp(0); idx.len() * self.rows];
        status(unsafe { hl_b200_store_columns(self.h, ix.as_ptr(), ix.len(), out.as_mut_ptr() as *mut u64) })?;
        Ok(out.chunks(self.rows.max(1)).map(|c| c.to_vec()).collect())
    }
    /// one pass over the resident data serves every vector
    fn fold_batch(&self) -> usize {
        usize::MAX
    }
    /// the pads are the commitment's own, resident beside the data rows
    fn fold_rows_with_pads(&self, rhos: &[Vec<Fp2>], _pads: &[Fp], q: usize) -> Option<Result<Vec<Vec<Fp2>>, String>> {
        (q == self.q).then(|| self.fold(rhos, 1, self.n + q))
    }
}

/// The signed byte width that holds every word of a row exactly (gpu/cuda.rs:903-910): 1, 2, 4, or 8 for a full word.
fn row_width(row: &[Fp]) -> u8 {
    const P: u64 = 0xFFFF_FFFF_0000_0001;
    let mut w = 1u8;
    for v in row {
        let v = v.0;
        let c = if v <= 0x7F || v >= P - 0x80 {
            1
        } else if v <= 0x7FFF || v >= P - 0x8000 {
            2
        } else if v <= 0x7FFF_FFFF || v >= P - 0x8000_0000 {
            4
        } else {
            return 8;
        };
        w = w.max(c);
    }
    w
}

/// rows packed at their own widths for `hl_b200_commit_zk_packed` (two's complement, little endian; gpu/cuda.rs:926-960)
fn pack_rows(data: &[Fp], n: usize) -> (Vec<u8>, Vec<u8>) {
    const P: u64 = 0xFFFF_FFFF_0000_0001;
    let widths: Vec<u8> = data.chunks(n).map(row_width).collect();
    let mut out = Vec::with_capacity(widths.iter().map(|&w| w as usize * n).sum());
    for (row, &w) in data.chunks(n).zip(widths.iter()) {
        for v in row {
            let x = if w == 8 || v.0 < (1u64 << 63) { v.0 } else { v.0.wrapping_sub(P) };
            out.extend_from_slice(&x.to_le_bytes()[..w as usize]);
        }
    }
    (out, widths)
}

pub struct B200Backend;

impl B200Backend {
    fn zk(&self, p: &PcsParams, data: &[Fp], pads: &[Fp], pows: &[Fp], ntt: &NttTables, key: Option<&[u8; 32]>) -> Option<(B200Commit, Vec<Digest>)> {
        if !enabled() {
            return None;
        }
        let (n, nn) = (p.cols(), p.enc_cols());
        if n == 0 || data.len() % n != 0 || data.is_empty() {
            return None;
        }
        let rows = data.len() / n;
        let q = pads.len() / rows;
        let mut leaves = vec![[0u8; 32]; nn];
        let mut h: *mut HlStore = std::ptr::null_mut();
        let key_ptr = key.map(|k| k.as_ptr()).unwrap_or(std::ptr::null());
        // narrow witness planes travel as their bytes (the reference's CUDA uploader does the same, gpu/mod.rs:270-300)
        let narrow = std::env::var("HL_GPU_NARROW").map(|v| v != "0").unwrap_or(true) && p.log_cols >= 3;
        let rc = if narrow {
            let (packed, widths) = pack_rows(data, n);
            unsafe {
                hl_b200_commit_zk_packed(ctx(), p.log_cols, p.inv_rate as u32, packed.as_ptr() as *const c_void, widths.as_ptr(), rows, words(pads), q,
                                         words(pows), ntt.max_log, key_ptr, std::ptr::null(), std::ptr::null(), std::ptr::null(), &mut h,
                                         leaves.as_mut_ptr() as *mut u8, std::ptr::null_mut())
            }
        } else {
            unsafe {
                hl_b200_commit_zk(ctx(), p.log_cols, p.inv_rate as u32, words(data), rows, words(pads), q, words(pows), ntt.max_log, key_ptr, &mut h,
                                  leaves.as_mut_ptr() as *mut u8)
            }
        };
        if rc != 0 {
            super::declined("[ZK60-B200] zk commit", &last_error());
            return None;
        }
        Some((B200Commit { h, rows, n, q }, leaves))
    }
}

/// What the device found wrong with an opened column (pcs.rs:1313-1327).
pub enum ColumnVerdict {
    MerklePath(usize),
    Disagrees { column: usize, vector: usize },
}

/// The map over the opened columns of `verify_zk_tagged` (pcs.rs:1282-1331) on the device, the encoding of the clear vectors
/// included.  `vecs`: the group vectors then the proximity vector, `n + q` entries each; `rhos`: their combined row weights in the
/// same order; the caller has already checked path lengths, column lengths and `j == want_j`.  `Ok(None)`: every column passes;
/// `Ok(Some(v))`: the first failing column; `Err`: the device declined and the host body runs.
/// (A caller that keeps a device commitment of the vectors' rows uses `hl_b200_verify_columns` with that store instead.)
#[allow(clippy::too_many_arguments)]
pub fn verify_columns(p: &PcsParams, q: usize, pows: &[Fp], root: &Digest, keys: [Option<&[u8; 32]>; 3], rhos: &[Vec<Fp2>], vecs: &[&Vec<Fp2>],
                      columns: &[(usize, Vec<Fp>, [u8; 32], Vec<Digest>)]) -> Result<Option<ColumnVerdict>, String> {
    let rows = columns.first().map(|c| c.1.len()).unwrap_or(0);
    if !enabled() || rows == 0 || vecs.len() != rhos.len() {
        return Err("b200 verify: nothing to do on the device".into());
    }
    let depth = columns[0].3.len();
    let mut cols = Vec::with_capacity(columns.len() * rows);
    let mut idx = Vec::with_capacity(columns.len());
    let mut salts = Vec::with_capacity(columns.len() * 32);
    let mut paths = Vec::with_capacity(columns.len() * depth * 32);
    for (j, col, salt, path) in columns {
        idx.push(*j as u64);
        cols.extend_from_slice(col);
        salts.extend_from_slice(salt);
        for d in path {
            paths.extend_from_slice(d);
        }
    }
    let flat_v: Vec<Fp2> = vecs.iter().flat_map(|v| v.iter().copied()).collect();
    let flat_r: Vec<Fp2> = rhos.iter().flat_map(|r| r.iter().copied()).collect();
    let kp = |k: Option<&[u8; 32]>| k.map(|x| x.as_ptr()).unwrap_or(std::ptr::null());
    let mut verdict = vec![0i32; columns.len()];
    let mut first: i64 = -1;
    status(unsafe {
        hl_b200_verify_opening(ctx(), p.log_cols, p.inv_rate as u32, q, words(pows), flat_v.as_ptr() as *const u64, vecs.len(), words(&cols), rows,
                               columns.len(), idx.as_ptr(), salts.as_ptr(), paths.as_ptr(), depth as u32, root.as_ptr(), kp(keys[0]), kp(keys[1]),
                               kp(keys[2]), flat_r.as_ptr() as *const u64, verdict.as_mut_ptr(), &mut first)
    })?;
    Ok(if first < 0 {
        None
    } else if verdict[first as usize] == 1 {
        Some(ColumnVerdict::MerklePath(columns[first as usize].0))
    } else {
        Some(ColumnVerdict::Disagrees { column: columns[first as usize].0, vector: (verdict[first as usize] - 2) as usize })
    })
}

impl Backend for B200Backend {
    type Store = B200Commit;
    fn try_commit(&self, p: &PcsParams, data: &[Fp], ntt: &NttTables) -> Option<(B200Commit, Vec<Digest>)> {
        if !enabled() {
            return None;
        }
        let (n, nn) = (p.cols(), p.enc_cols());
        if n == 0 || data.is_empty() || data.len() % n != 0 {
            return None;
        }
        let rows = data.len() / n;
        let mut leaves = vec![[0u8; 32]; nn];
        let mut h: *mut HlStore = std::ptr::null_mut();
        let rc = unsafe {
            hl_b200_commit(ctx(), p.log_cols, p.inv_rate as u32, words(data), rows, ntt.max_log, std::ptr::null(), &mut h, leaves.as_mut_ptr() as *mut u8)
        };
        if rc != 0 {
            super::declined("[ZK60-B200] commit", &last_error());
            return None;
        }
        Some((B200Commit { h, rows, n, q: 0 }, leaves))
    }
    fn try_commit_zk(&self, p: &PcsParams, data: &[Fp], pads: &[Fp], pows: &[Fp], ntt: &NttTables) -> Option<(B200Commit, Vec<Digest>)> {
        self.zk(p, data, pads, pows, ntt, None)
    }
    fn try_commit_zk_keyed(&self, p: &PcsParams, data: &[Fp], pads: &[Fp], pows: &[Fp], ntt: &NttTables, key: &[u8; 32]) -> Option<(B200Commit, Vec<Digest>)> {
        self.zk(p, data, pads, pows, ntt, Some(key))
    }
}

/// The device evaluator of one sumcheck.  Deliberately not `Sync`: one evaluator belongs to one thread (rounds.rs:20-21).
pub struct B200Rounds {
    h: *mut HlRounds,
    n: usize,
    d: usize,
    k: usize,
}
impl Drop for B200Rounds {
    fn drop(&mut self) {
        unsafe { hl_b200_rounds_free(self.h) }
    }
}

/// The builtin polynomial families of include/hl_b200.h (`HL_POLY_*`).
pub const POLY_PROD: c_int = 0;
pub const POLY_ZC: c_int = 1;
pub const POLY_LOGUP_Q: c_int = 2;
pub const POLY_LOGUP_T: c_int = 3;

fn flat_tables(tables: &[Vec<Fp2>]) -> Vec<u64> {
    let mut flat = Vec::with_capacity(tables.len() * tables[0].len() * 2);
    for t in tables {
        for x in t {
            flat.push(x.c0.0);
            flat.push(x.c1.0);
        }
    }
    flat
}

impl B200Rounds {
    /// a builtin family over `tables` (each of 2^n_vars entries); `Ok(None)` = the device declines and the CPU evaluator runs
    pub fn builtin(poly: c_int, tables: &[Vec<Fp2>], degree: usize, coefs: &[Fp2]) -> Result<Option<B200Rounds>, String> {
        if !enabled() || tables.is_empty() {
            return Ok(None);
        }
        let n = tables[0].len().trailing_zeros() as usize;
        let cf: Vec<u64> = coefs.iter().flat_map(|c| [c.c0.0, c.c1.0]).collect();
        let mut h: *mut HlRounds = std::ptr::null_mut();
        let rc = unsafe {
            hl_b200_rounds_new(ctx(), poly, tables.len(), n as u32, degree as u32, flat_tables(tables).as_ptr(), cf.as_ptr(), coefs.len(), &mut h)
        };
        if rc != 0 {
            super::declined("[ZK60-B200] rounds", &last_error());
            return Ok(None);
        }
        Ok(Some(B200Rounds { h, n, d: degree, k: tables.len() }))
    }

    /// any slot polynomial, given as its expression graph (private_block/slot_ir.rs:57-345) flattened into the word stream of
    /// include/hl_b200.h: the nodes in order, then the terms; a coefficient equal to 1, -1 or 0 is a special word, every
    /// other value goes to the coefficient array
    pub fn from_ir(ir: &crate::private_block::slot_ir::SlotIr, tables: &[Vec<Fp2>], degree: usize) -> Result<Option<B200Rounds>, String> {
        use crate::private_block::slot_ir::{Factor, NodeBody};
        if !enabled() || tables.is_empty() {
            return Ok(None);
        }
        const ONE: u32 = 0xFFFF_FFFF;
        const NEG_ONE: u32 = 0xFFFF_FFFE;
        const ZERO: u32 = 0xFFFF_FFFD;
        const NODE: u32 = 0x8000_0000;
        let mut words: Vec<u32> = Vec::new();
        let mut coefs: Vec<u64> = Vec::new();
        let mut coef = |v: Fp2| -> u32 {
            if v == Fp2::ONE {
                ONE
            } else if v == Fp2::ZERO.sub(Fp2::ONE) {
                NEG_ONE
            } else if v == Fp2::ZERO {
                ZERO
            } else {
                coefs.push(v.c0.0);
                coefs.push(v.c1.0);
                (coefs.len() / 2 - 1) as u32
            }
        };
        let fac = |f: &Factor| match f {
            Factor::Table(t) => *t as u32,
            Factor::Node(n) => NODE | *n as u32,
        };
        for node in &ir.nodes {
            match &node.body {
                NodeBody::Affine { konst, terms } => {
                    words.push((terms.len() as u32) << 8);
                    words.push(coef(konst.value));
                    for (c, t) in terms {
                        words.push(coef(c.value));
                        words.push(*t as u32);
                    }
                }
                NodeBody::Sum { subterms } => {
                    words.push(1 | (subterms.len() as u32) << 8);
                    for s in subterms {
                        words.push(coef(s.coef.value));
                        words.push(s.factors.len() as u32);
                        words.extend(s.factors.iter().map(fac));
                    }
                }
            }
        }
        for t in &ir.terms {
            words.push(coef(t.coef.value));
            words.push((t.wrapper.len() + t.inner.len()) as u32);
            words.extend(t.wrapper.iter().map(|x| *x as u32));
            words.extend(t.inner.iter().map(fac));
        }
        let n = tables[0].len().trailing_zeros() as usize;
        let mut h: *mut HlRounds = std::ptr::null_mut();
        let rc = unsafe {
            hl_b200_rounds_new_ir(ctx(), tables.len(), n as u32, degree as u32, flat_tables(tables).as_ptr(), words.as_ptr(), words.len(),
                                  ir.nodes.len() as u32, ir.terms.len() as u32, coefs.as_ptr(), coefs.len() / 2, &mut h)
        };
        if rc != 0 {
            super::declined("[ZK60-B200] slot rounds", &last_error());
            return Ok(None);
        }
        Ok(Some(B200Rounds { h, n, d: degree, k: tables.len() }))
    }
}

impl SumcheckRounds for B200Rounds {
    fn n_vars(&self) -> usize {
        self.n
    }
    fn degree(&self) -> usize {
        self.d
    }
    fn round(&mut self, j: usize) -> Vec<Fp2> {
        let mut out = vec![0u64; (self.d + 1) * 2];
        let rc = unsafe { hl_b200_rounds_round(self.h, j as u32, 1, out.as_mut_ptr()) };
        assert_eq!(rc, 0, "[ZK60-B200] round {j}: {}", last_error());  // the trait has no error path: a device failure mid-sumcheck is fatal, as on Metal
        out.chunks(2).map(|w| Fp2 { c0: Fp(w[0]), c1: Fp(w[1]) }).collect()
    }
    fn fold(&mut self, r: Fp2) {
        let rr = [r.c0.0, r.c1.0];
        let rc = unsafe { hl_b200_rounds_fold(self.h, rr.as_ptr()) };
        assert_eq!(rc, 0, "[ZK60-B200] fold: {}", last_error());
    }
    fn finals(&self) -> Vec<Fp2> {
        let mut out = vec![0u64; self.k * 2];
        let rc = unsafe { hl_b200_rounds_finals(self.h, out.as_mut_ptr()) };
        assert_eq!(rc, 0, "[ZK60-B200] finals: {}", last_error());
        out.chunks(2).map(|w| Fp2 { c0: Fp(w[0]), c1: Fp(w[1]) }).collect()
    }
}
