//! Safetensors files: `model.save(Format::Safetensors, path)` / `load_safetensors(path)`.
//!
//! The container is the plain safetensors layout (8-byte little-endian header length, a JSON header mapping tensor
//! names to `dtype`, `shape` and `data_offsets`, then the raw little-endian data), written to a temporary file and
//! renamed into place, as the Python package does (`incin_b200/io/safetensors.py`) and as the reference does
//! (crates/incin-core/src/nn/save.rs).  Tensor names follow the flat module numbering of both (`0.weight`, `0.bias`,
//! `2.weight`, ... for a sequential model), so a file written here loads there and vice versa.  Only fp32 is written;
//! fp32 is what this crate's CPU backend holds.
use std::fs;
use std::io::{self, Read, Write};
use std::path::Path;

use crate::nn::Mlp;

/// Storage formats of `save`.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Format {
    Safetensors,
}

/// One named fp32 tensor of a file.
#[derive(Debug, Clone, PartialEq)]
pub struct NamedTensor {
    pub name: String,
    pub shape: Vec<usize>,
    pub data: Vec<f32>,
}

fn bad(msg: &str) -> io::Error {
    io::Error::new(io::ErrorKind::InvalidData, msg.to_string())
}

/// Write `tensors` in the given order.  The header is padded with spaces to a multiple of 8 bytes.
pub fn save_safetensors(path: &Path, tensors: &[NamedTensor]) -> io::Result<()> {
    let mut header = String::from("{");
    let mut offset = 0usize;
    for (i, t) in tensors.iter().enumerate() {
        let count: usize = t.shape.iter().product();
        if count != t.data.len() || t.name.contains('"') || t.name.contains('\\') {
            return Err(bad("tensor name or shape does not fit its data"));
        }
        if i > 0 {
            header.push(',');
        }
        let dims: Vec<String> = t.shape.iter().map(|d| d.to_string()).collect();
        let end = offset + 4 * count;
        header.push_str(&format!("\"{}\":{{\"dtype\":\"F32\",\"shape\":[{}],\"data_offsets\":[{},{}]}}", t.name,
                                 dims.join(","), offset, end));
        offset = end;
    }
    header.push('}');
    while header.len() % 8 != 0 {
        header.push(' ');
    }
    let tmp = path.with_extension("safetensors.tmp");
    {
        let mut f = fs::File::create(&tmp)?;
        f.write_all(&(header.len() as u64).to_le_bytes())?;
        f.write_all(header.as_bytes())?;
        for t in tensors {
            for v in &t.data {
                f.write_all(&v.to_le_bytes())?;
            }
        }
        f.sync_all()?;
    }
    fs::rename(&tmp, path)
}

// ---- the small part of JSON a safetensors header uses ------------------------------------------------------
struct Cursor<'a> {
    s: &'a [u8],
    i: usize,
}

impl<'a> Cursor<'a> {
    fn ws(&mut self) {
        while self.i < self.s.len() && (self.s[self.i] as char).is_ascii_whitespace() {
            self.i += 1;
        }
    }

    fn eat(&mut self, c: u8) -> io::Result<()> {
        self.ws();
        if self.i < self.s.len() && self.s[self.i] == c {
            self.i += 1;
            Ok(())
        } else {
            Err(bad("malformed safetensors header"))
        }
    }

    fn peek(&mut self) -> Option<u8> {
        self.ws();
        self.s.get(self.i).copied()
    }

    fn string(&mut self) -> io::Result<String> {
        self.eat(b'"')?;
        let start = self.i;
        while self.i < self.s.len() && self.s[self.i] != b'"' {
            if self.s[self.i] == b'\\' {
                return Err(bad("escaped characters in tensor names are not supported"));
            }
            self.i += 1;
        }
        let out = String::from_utf8(self.s[start..self.i.min(self.s.len())].to_vec()).map_err(|_| bad("name is not utf-8"))?;
        self.eat(b'"')?;
        Ok(out)
    }

    fn number(&mut self) -> io::Result<usize> {
        self.ws();
        let start = self.i;
        while self.i < self.s.len() && self.s[self.i].is_ascii_digit() {
            self.i += 1;
        }
        if start == self.i {
            return Err(bad("expected a non-negative integer"));
        }
        std::str::from_utf8(&self.s[start..self.i]).ok().and_then(|t| t.parse::<usize>().ok()).ok_or_else(|| bad("bad integer"))
    }

    fn numbers(&mut self) -> io::Result<Vec<usize>> {
        self.eat(b'[')?;
        let mut out = Vec::new();
        if self.peek() == Some(b']') {
            self.i += 1;
            return Ok(out);
        }
        loop {
            out.push(self.number()?);
            match self.peek() {
                Some(b',') => self.i += 1,
                Some(b']') => {
                    self.i += 1;
                    return Ok(out);
                }
                _ => return Err(bad("malformed array")),
            }
        }
    }

    /// Skip one value of an entry this reader does not interpret (`__metadata__`: an object of strings).
    fn skip_object_of_strings(&mut self) -> io::Result<()> {
        self.eat(b'{')?;
        if self.peek() == Some(b'}') {
            self.i += 1;
            return Ok(());
        }
        loop {
            self.string()?;
            self.eat(b':')?;
            self.string()?;
            match self.peek() {
                Some(b',') => self.i += 1,
                Some(b'}') => {
                    self.i += 1;
                    return Ok(());
                }
                _ => return Err(bad("malformed metadata")),
            }
        }
    }
}

/// Read every fp32 tensor of a safetensors file, in file order of the header.
pub fn load_safetensors(path: &Path) -> io::Result<Vec<NamedTensor>> {
    let mut bytes = Vec::new();
    fs::File::open(path)?.read_to_end(&mut bytes)?;
    if bytes.len() < 8 {
        return Err(bad("file shorter than its header length"));
    }
    let mut len8 = [0u8; 8];
    len8.copy_from_slice(&bytes[..8]);
    let hlen = u64::from_le_bytes(len8) as usize;
    if hlen > bytes.len() - 8 {
        return Err(bad("header length exceeds the file"));
    }
    let data = &bytes[8 + hlen..];
    let mut c = Cursor { s: &bytes[8..8 + hlen], i: 0 };
    let mut out = Vec::new();
    c.eat(b'{')?;
    if c.peek() == Some(b'}') {
        return Ok(out);
    }
    loop {
        let name = c.string()?;
        c.eat(b':')?;
        if name == "__metadata__" {
            c.skip_object_of_strings()?;
        } else {
            c.eat(b'{')?;
            let (mut dtype, mut shape, mut offsets) = (String::new(), Vec::new(), Vec::new());
            loop {
                let key = c.string()?;
                c.eat(b':')?;
                match key.as_str() {
                    "dtype" => dtype = c.string()?,
                    "shape" => shape = c.numbers()?,
                    "data_offsets" => offsets = c.numbers()?,
                    _ => return Err(bad("unknown key in a tensor entry")),
                }
                match c.peek() {
                    Some(b',') => c.i += 1,
                    Some(b'}') => {
                        c.i += 1;
                        break;
                    }
                    _ => return Err(bad("malformed tensor entry")),
                }
            }
            if dtype != "F32" {
                return Err(bad("only F32 tensors are read by this crate"));
            }
            let count: usize = shape.iter().product();
            if offsets.len() != 2 || offsets[1] < offsets[0] || offsets[1] - offsets[0] != 4 * count || offsets[1] > data.len() {
                return Err(bad("data offsets do not match the shape"));
            }
            let mut values = Vec::with_capacity(count);
            for chunk in data[offsets[0]..offsets[1]].chunks_exact(4) {
                values.push(f32::from_le_bytes([chunk[0], chunk[1], chunk[2], chunk[3]]));
            }
            out.push(NamedTensor { name, shape, data: values });
        }
        match c.peek() {
            Some(b',') => c.i += 1,
            Some(b'}') => return Ok(out),
            _ => return Err(bad("malformed header")),
        }
    }
}

impl Mlp {
    /// The model's tensors under the flat sequential numbering (`0` = first linear, `1` = ReLU, `2` = second linear).
    pub fn state_dict(&self) -> Vec<NamedTensor> {
        let l = |name: &str, shape: Vec<usize>, data: &Vec<f32>| NamedTensor { name: name.to_string(), shape, data: data.clone() };
        vec![
            l("0.weight", vec![self.fc1.out_features, self.fc1.in_features], &self.fc1.weight),
            l("0.bias", vec![self.fc1.out_features], &self.fc1.bias),
            l("2.weight", vec![self.fc2.out_features, self.fc2.in_features], &self.fc2.weight),
            l("2.bias", vec![self.fc2.out_features], &self.fc2.bias),
        ]
    }

    pub fn save(&self, format: Format, path: &Path) -> io::Result<()> {
        match format {
            Format::Safetensors => save_safetensors(path, &self.state_dict()),
        }
    }

    /// Load tensors by name; shapes must match the model that was built.
    pub fn load(&mut self, path: &Path) -> io::Result<()> {
        let want = self.state_dict();
        let got = load_safetensors(path)?;
        for w in &want {
            let t = got.iter().find(|t| t.name == w.name).ok_or_else(|| bad("a tensor of the model is missing from the file"))?;
            if t.shape != w.shape {
                return Err(bad("a tensor in the file has a different shape than the model"));
            }
        }
        let take = |name: &str| got.iter().find(|t| t.name == name).map(|t| t.data.clone()).unwrap_or_default();
        self.fc1.weight = take("0.weight");
        self.fc1.bias = take("0.bias");
        self.fc2.weight = take("2.weight");
        self.fc2.bias = take("2.bias");
        Ok(())
    }
}
