//! Wire format of the B200 backend's C-ABI (`include/adb200.h`): `IRProcedure` + dep list -> one flat blob.
//!
//! Written for the reference tree (drop into `src/devices/cuda/`); NOT COMPILED HERE -- the environment this backend
//! was built in has no Rust toolchain.  The byte layout is pinned by fixtures produced by the Python twin of this
//! file (`autodiff-ir-rust_b200/ir.py`): `tests/golden/wire/*.adir`; the test at the bottom rebuilds the
//! `all_variants` program with the reference's own types and compares byte for byte.
//!
//! Layout (little-endian, version 1):
//!   u32 magic 'ADIR' | u32 version | u32 flags | u32 n_ids | n_ids x { u16 len, bytes }
//!   u32 n_dep | n_dep x u32 (indices into the id table, ids sorted)
//!   procedure := u32 n_cmds, n_cmds x cmd        cmd := u8 opcode, operands
//!   payload section: f32 data of inline CreateMat payloads, each 16-byte aligned
//! Ids get their index in the table at their first appearance during the walk (dep-list ids last).
use std::collections::{HashMap, HashSet};

use crate::{IRCmds, IRProcedure};

pub const MAGIC: u32 = 0x5249_4441; // 'ADIR'
pub const VERSION: u32 = 1;

/// How `CreateMat` contents travel: copied into the blob, or passed by host address (zero copy; the `Arc<Vec<f32>>`
/// must outlive `adb_execute`, which it does: the IR holds it).
#[derive(Clone, Copy, PartialEq)]
pub enum Payloads {
    Inline,
    /// by address above this many bytes, inline below
    HostPointersAbove(usize),
}

const PAYLOAD_INLINE: u8 = 0;
const PAYLOAD_HOST: u8 = 1;

struct Writer {
    ids: HashMap<String, u32>,
    order: Vec<String>,
    body: Vec<u8>,
    inline: Vec<(usize, std::sync::Arc<Vec<f32>>)>, // (position of the u64 to patch, data)
    payloads: Payloads,
}

impl Writer {
    fn idx(&mut self, s: &str) -> u32 {
        if let Some(&i) = self.ids.get(s) {
            return i;
        }
        let i = self.order.len() as u32;
        self.ids.insert(s.to_string(), i);
        self.order.push(s.to_string());
        i
    }
    fn u8(&mut self, v: u8) { self.body.push(v) }
    fn u16(&mut self, v: u16) { self.body.extend_from_slice(&v.to_le_bytes()) }
    fn u32(&mut self, v: u32) { self.body.extend_from_slice(&v.to_le_bytes()) }
    fn u64(&mut self, v: u64) { self.body.extend_from_slice(&v.to_le_bytes()) }
    fn f32(&mut self, v: f32) { self.body.extend_from_slice(&v.to_le_bytes()) }
    fn id(&mut self, s: &str) { let i = self.idx(s); self.u32(i) }
    fn dims(&mut self, d: &[usize]) {
        self.u8(d.len() as u8);
        for &x in d { self.u64(x as u64) }
    }
    fn proc(&mut self, p: &IRProcedure) {
        self.u32(p.main.len() as u32);
        for c in &p.main { self.cmd(c) }
    }
    fn cmd(&mut self, c: &IRCmds) {
        match c {
            IRCmds::CreateMat { contents, dim, id } => {
                self.u8(1); self.id(id); self.dims(dim);
                let bytes = contents.len() * 4;
                let by_address = matches!(self.payloads, Payloads::HostPointersAbove(limit) if bytes > limit);
                if by_address {
                    self.u8(PAYLOAD_HOST);
                    self.u64(contents.as_ptr() as u64);
                } else {
                    self.u8(PAYLOAD_INLINE);
                    self.inline.push((self.body.len(), contents.clone()));
                    self.u64(0);
                }
                self.u64(contents.len() as u64);
            }
            IRCmds::CreateConstant { contents, id, dim } => { self.u8(2); self.id(id); self.f32(*contents); self.dims(dim) }
            IRCmds::ElwMultiply { a, b, res } => { self.u8(3); self.id(a); self.id(b); self.id(res) }
            IRCmds::ElwAdd { a, b, res } => { self.u8(4); self.id(a); self.id(b); self.id(res) }
            IRCmds::ElwMultiplyEq { s, o } => { self.u8(5); self.id(s); self.id(o) }
            IRCmds::ElwAddEq { s, o } => { self.u8(6); self.id(s); self.id(o) }
            IRCmds::EqualZero { a, res } => { self.u8(7); self.id(a); self.id(res) }
            IRCmds::MoreZero { a, res } => { self.u8(8); self.id(a); self.id(res) }
            IRCmds::LessZero { a, res } => { self.u8(9); self.id(a); self.id(res) }
            IRCmds::Sum { a, res } => { self.u8(10); self.id(a); self.id(res) }
            IRCmds::DotProduct { a, b, res } => { self.u8(11); self.id(a); self.id(b); self.id(res) }
            IRCmds::View { a, target_dim, res } => { self.u8(12); self.id(a); self.id(res); self.dims(target_dim) }
            IRCmds::Index { a, index, dim, res } => { self.u8(13); self.id(a); self.id(res); self.u64(*index as u64); self.u32(*dim as u32) }
            IRCmds::Concat { a, b, dim, res } => { self.u8(14); self.id(a); self.id(b); self.id(res); self.u32(*dim as u32) }
            IRCmds::Permute { a, p, res } => {
                self.u8(15); self.id(a); self.id(res); self.u8(p.len() as u8);
                for &x in p { self.u32(x as u32) }
            }
            IRCmds::Broadcast { a, dim, r, res } => { self.u8(16); self.id(a); self.id(res); self.u32(*dim as u32); self.u64(*r as u64) }
            IRCmds::Contigious { a, res } => { self.u8(17); self.id(a); self.id(res) }
            IRCmds::Exp2 { a, res } => { self.u8(18); self.id(a); self.id(res) }
            IRCmds::Log2 { a, res } => { self.u8(19); self.id(a); self.id(res) }
            IRCmds::Sin { a, res } => { self.u8(20); self.id(a); self.id(res) }
            IRCmds::Recip { a, res } => { self.u8(21); self.id(a); self.id(res) }
            IRCmds::Sqrt { a, res } => { self.u8(22); self.id(a); self.id(res) }
            IRCmds::While { conditional_var, block } => { self.u8(23); self.id(conditional_var); self.proc(block) }
            IRCmds::If { conditions, else_proc } => {
                self.u8(24);
                self.u32(conditions.len() as u32);
                for (cond, blk) in conditions { self.id(cond); self.proc(blk) }
                match else_proc {
                    None => self.u8(0),
                    Some(p) => { self.u8(1); self.proc(p) }
                }
            }
            IRCmds::EX => self.u8(25),
            IRCmds::Heading { cmt } => {
                let b = cmt.as_bytes();
                let n = b.len().min(65535);
                self.u8(26); self.u16(n as u16); self.body.extend_from_slice(&b[..n]);
            }
        }
    }
}

/// `proc` (nested blocks included) and the ids that must be readable afterwards (`core::ret_dep_list()`) as one blob
/// for `adb_execute`.  With `Payloads::HostPointersAbove` the blob borrows the `CreateMat` vectors: keep `proc` alive
/// until `adb_execute` has returned.
pub fn serialize(proc: &IRProcedure, dep: &HashSet<String>, payloads: Payloads) -> Vec<u8> {
    let mut w = Writer { ids: HashMap::new(), order: Vec::new(), body: Vec::new(), inline: Vec::new(), payloads };
    w.proc(proc);
    let mut dep_sorted: Vec<&String> = dep.iter().collect();
    dep_sorted.sort();
    let dep_idx: Vec<u32> = dep_sorted.iter().map(|d| w.idx(d)).collect();

    let mut blob = Vec::with_capacity(w.body.len() + 64);
    for v in [MAGIC, VERSION, 0u32, w.order.len() as u32] { blob.extend_from_slice(&v.to_le_bytes()) }
    for s in &w.order {
        blob.extend_from_slice(&(s.len() as u16).to_le_bytes());
        blob.extend_from_slice(s.as_bytes());
    }
    blob.extend_from_slice(&(dep_idx.len() as u32).to_le_bytes());
    for i in dep_idx { blob.extend_from_slice(&i.to_le_bytes()) }
    let body_off = blob.len();
    blob.extend_from_slice(&w.body);
    // payload section, each payload 16-byte aligned; its byte offset is patched into the command
    for (pos, data) in &w.inline {
        while blob.len() % 16 != 0 { blob.push(0) }
        let off = blob.len() as u64;
        blob[body_off + pos..body_off + pos + 8].copy_from_slice(&off.to_le_bytes());
        for v in data.iter() { blob.extend_from_slice(&v.to_le_bytes()) }
    }
    blob
}

#[cfg(test)]
mod tests {
    use super::*;
    use std::sync::Arc;

    fn p(id: &str, cmds: Vec<IRCmds>) -> IRProcedure { IRProcedure { main: cmds, id: id.to_string() } }
    fn s(x: &str) -> String { x.to_string() }

    /// Every `IRCmds` variant once, nested blocks included; `tests/golden/make_wire_fixtures.py` builds the same
    /// program with the Python serialiser and commits its bytes.
    #[test]
    fn all_variants_match_the_committed_bytes() {
        let body = p("b0", vec![
            IRCmds::ElwAddEq { s: s("c"), o: s("k") },
            IRCmds::If {
                conditions: vec![(s("f"), p("b1", vec![IRCmds::ElwMultiplyEq { s: s("a"), o: s("a") }])),
                                 (s("g"), p("b2", vec![IRCmds::EX]))],
                else_proc: Some(p("b3", vec![IRCmds::Heading { cmt: s("else") }])),
            },
        ]);
        let main = p("main", vec![
            IRCmds::Heading { cmt: s("all variants") },
            IRCmds::CreateMat { contents: Arc::new(vec![1.0, 2.0, 3.0, 4.0, 5.0, 6.0]), dim: vec![2, 3], id: s("a") },
            IRCmds::CreateMat { contents: Arc::new(vec![2.0]), dim: vec![1], id: s("c") },
            IRCmds::CreateMat { contents: Arc::new(vec![1.0]), dim: vec![1], id: s("f") },
            IRCmds::CreateMat { contents: Arc::new(vec![0.0]), dim: vec![1], id: s("g") },
            IRCmds::CreateConstant { contents: -1.0, id: s("k"), dim: vec![1] },
            IRCmds::CreateConstant { contents: 0.5, id: s("h"), dim: vec![2, 3] },
            IRCmds::ElwMultiply { a: s("a"), b: s("h"), res: s("m") },
            IRCmds::ElwAdd { a: s("a"), b: s("m"), res: s("n") },
            IRCmds::EqualZero { a: s("n"), res: s("e0") },
            IRCmds::MoreZero { a: s("n"), res: s("e1") },
            IRCmds::LessZero { a: s("n"), res: s("e2") },
            IRCmds::Sum { a: s("n"), res: s("sm") },
            IRCmds::Permute { a: s("a"), p: vec![1, 0], res: s("at") },
            IRCmds::DotProduct { a: s("a"), b: s("at"), res: s("d") },
            IRCmds::View { a: s("a"), target_dim: vec![3, 2], res: s("v") },
            IRCmds::Index { a: s("a"), index: 1, dim: 0, res: s("i") },
            IRCmds::Concat { a: s("a"), b: s("n"), dim: 0, res: s("cc") },
            IRCmds::View { a: s("sm"), target_dim: vec![2, 1], res: s("s1") },
            IRCmds::Broadcast { a: s("s1"), dim: 1, r: 3, res: s("bc") },
            IRCmds::Contigious { a: s("at"), res: s("ct") },
            IRCmds::Exp2 { a: s("a"), res: s("u0") },
            IRCmds::Log2 { a: s("a"), res: s("u1") },
            IRCmds::Sin { a: s("a"), res: s("u2") },
            IRCmds::Recip { a: s("a"), res: s("u3") },
            IRCmds::Sqrt { a: s("a"), res: s("u4") },
            IRCmds::While { conditional_var: s("c"), block: body },
            IRCmds::EX,
        ]);
        let dep: HashSet<String> = ["a", "d", "cc", "bc", "ct", "u4", "c"].iter().map(|x| x.to_string()).collect();
        let blob = serialize(&main, &dep, Payloads::Inline);
        let want = include_bytes!("../../../../tests/golden/wire/all_variants.adir");
        assert_eq!(blob.as_slice(), &want[..]);
    }
}
