//! Walks `ModelDefinition.ir()` (crates/trainer/src/model/definition.rs:33-71,
//! crates/compiler/src/model.rs:137-161) and recognises the one family of graphs the B200
//! library runs: a shared sparse affine on both perspectives, CReLU / SCReLU or pairwise
//! CReLU, the stm|nstm concat, one to three output-bucketed dense layers and
//! `sigmoid().squared_error(targets)` summed over the batch.  Anything else is an `Err` that
//! names the operation that was not expected; nothing is ever trained "approximately".
//!
//! The IR exposes its operations as trait objects, so they are told apart by `opname()`
//! (crates/compiler/src/model/operations/*.rs): "Binary.Add", "Binary.Mul", "Matmul<..>",
//! "Sparse.Matmul<..>", "CReLU", "SCReLU", "Sigmoid", "Concat", "Select", "ReduceSum<Batch>",
//! "Broadcast<Batch>", "Broadcast<Cols, n>" (`repeat`), and — a quirk of the reference — a row
//! slice prints as "Pad<start, end, true>" (operations/index.rs:24-27).
use std::collections::BTreeMap;

use b200_sys::{B200_ACT_CRELU, B200_ACT_NONE, B200_ACT_SCRELU, b200_net_desc};
use bullet_compiler::{
    ir::NodeId,
    model::{Layout, MType, ModelIR},
};
use bullet_trainer::model::ModelDefinition;

/// What the graph turned out to be, in the terms of `b200_net_create`.
#[derive(Clone, Debug)]
pub struct Recognised {
    pub desc: b200_net_desc,
    /// (weight id in the graph, tensor name at the C ABI): l0w, l0b, [l0f], l1w, l1b, ...
    pub weights: Vec<(String, &'static str)>,
    /// names of the graph inputs that feed the two perspectives, the output buckets and the targets
    pub stm: String,
    pub ntm: String,
    pub buckets: Option<String>,
    pub targets: String,
}

struct Walk<'a> {
    ir: &'a ModelIR,
}

/// One step up from a node: the name of the operation that made it and that operation's inputs.
struct Made {
    name: String,
    inputs: Vec<NodeId>,
}

impl<'a> Walk<'a> {
    fn made(&self, node: NodeId) -> Result<Made, String> {
        let inner = self.ir.inner();
        let id = inner.parent_op(node).map_err(|e| format!("{e}"))?;
        let op = inner.op(id).map_err(|e| format!("{e}"))?;
        Ok(Made { name: op.data().0.opname(), inputs: op.inputs().to_vec() })
    }

    fn ty(&self, node: NodeId) -> MType {
        self.ir.node(node).ty()
    }

    /// `binary()` broadcasts the unbatched side across the batch (builder.rs:263-267): look through it.
    fn unbroadcast(&self, node: NodeId) -> Result<NodeId, String> {
        let m = self.made(node)?;
        Ok(if m.name.starts_with("Broadcast<Batch") { m.inputs[0] } else { node })
    }

    fn weight(&self, node: NodeId) -> Option<&'a str> {
        self.ir.weights().get(&node).map(|(name, _)| name.as_str())
    }

    fn input(&self, node: NodeId) -> Option<&'a str> {
        self.ir.inputs().get(&node).map(String::as_str)
    }

    /// "Pad<start, end, true>" -> (start, end)
    fn row_slice(name: &str) -> Option<(usize, usize)> {
        let body = name.strip_prefix("Pad<")?.strip_suffix('>')?;
        let mut parts = body.split(", ");
        let start = parts.next()?.parse().ok()?;
        let end = parts.next()?.parse().ok()?;
        (parts.next()? == "true").then_some((start, end))
    }

    /// `weights.matmul(x) + bias` (builder.rs:145-147) -> (weights node, bias node, x)
    fn affine(&self, node: NodeId) -> Result<(NodeId, NodeId, NodeId), String> {
        let add = self.made(node)?;
        if add.name != "Binary.Add" {
            return Err(format!("expected `weights.matmul(x) + bias`, found {}", add.name));
        }
        for (mm, bias) in [(add.inputs[0], add.inputs[1]), (add.inputs[1], add.inputs[0])] {
            let m = self.made(mm)?;
            if m.name.starts_with("Matmul<") || m.name.starts_with("Sparse.Matmul<") {
                return Ok((m.inputs[0], self.unbroadcast(bias)?, m.inputs[1]));
            }
        }
        Err("an addition whose operands are not a matmul and a bias (skip connections are not recognised)".into())
    }
}

#[derive(Clone, Debug, PartialEq)]
struct FtHalf {
    l0w: NodeId,
    l0f: Option<NodeId>,
    l0b: NodeId,
    input: NodeId,
    act: i32,
    pairwise: bool,
    rows: usize,
}

impl<'a> Walk<'a> {
    /// The table is `l0w`, or `l0w + l0f.repeat(n)` (examples/progression/4_multi_layer.rs:67-70).
    fn table(&self, node: NodeId) -> Result<(NodeId, Option<NodeId>), String> {
        if self.weight(node).is_some() {
            return Ok((node, None));
        }
        let add = self.made(node)?;
        if add.name == "Binary.Add" {
            for (w, rep) in [(add.inputs[0], add.inputs[1]), (add.inputs[1], add.inputs[0])] {
                let r = self.made(rep)?;
                if self.weight(w).is_some() && r.name.starts_with("Broadcast<Cols") && self.weight(r.inputs[0]).is_some() {
                    let (wt, ft) = (self.ty(w).shape(), self.ty(r.inputs[0]).shape());
                    if ft.rows() != wt.rows() || wt.cols() % ft.cols() != 0 {
                        return Err("factoriser: l0f.repeat(n) does not tile l0w".into());
                    }
                    return Ok((w, Some(r.inputs[0])));
                }
            }
        }
        Err(format!("feature transformer: weights are neither a weight nor weight + weight.repeat(n) ({})", add.name))
    }

    /// Strips `slice_rows(start, end)` from a weight expression; Err unless it is exactly that slice.
    fn sliced(&self, node: NodeId, start: usize, end: usize, what: &str) -> Result<NodeId, String> {
        let m = self.made(node)?;
        match Self::row_slice(&m.name) {
            Some((s, e)) if s == start && e == end => Ok(m.inputs[0]),
            _ => Err(format!("pairwise: expected rows {start}..{end} of the {what}, found {}", m.name)),
        }
    }

    fn ft_half(&self, node: NodeId) -> Result<FtHalf, String> {
        let top = self.made(node)?;
        let act = |name: &str| match name {
            "CReLU" => Some(B200_ACT_CRELU),
            "SCReLU" => Some(B200_ACT_SCRELU),
            _ => None,
        };
        if let Some(act) = act(&top.name) {
            let (w, b, x) = self.affine(top.inputs[0])?;
            let (l0w, l0f) = self.table(w)?;
            return Ok(FtHalf { l0w, l0f, l0b: b, input: x, act, pairwise: false, rows: self.ty(l0w).shape().rows() });
        }
        if top.name != "Binary.Mul" {
            return Err(format!("feature transformer: expected crelu/screlu of an affine layer or their pairwise product, found {}", top.name));
        }
        let (l, r) = (self.made(top.inputs[0])?, self.made(top.inputs[1])?);
        // spelling 1: l0.forward(x).crelu().pairwise_mul()  (builder.rs:390-393)
        if let (Some((ls, le)), Some((rs, re))) = (Self::row_slice(&l.name), Self::row_slice(&r.name)) {
            if l.inputs[0] != r.inputs[0] || self.made(l.inputs[0])?.name != "CReLU" {
                return Err("pairwise_mul must follow crelu()".into());
            }
            let rows = self.ty(l.inputs[0]).shape().rows();
            if (ls, le, rs, re) != (0, rows / 2, rows / 2, rows) || rows % 2 != 0 {
                return Err("pairwise_mul: the two halves of the rows were expected".into());
            }
            let (w, b, x) = self.affine(self.made(l.inputs[0])?.inputs[0])?;
            let (l0w, l0f) = self.table(w)?;
            return Ok(FtHalf { l0w, l0f, l0b: b, input: x, act: B200_ACT_CRELU, pairwise: true, rows });
        }
        // spelling 2: l0.slice(0, h/2).forward(x).crelu() * l0.slice(h/2, h).forward(x).crelu()
        // (examples/progression/4_multi_layer.rs:79-81)
        if l.name == "CReLU" && r.name == "CReLU" {
            let (w0, b0, x0) = self.affine(l.inputs[0])?;
            let (w1, b1, x1) = self.affine(r.inputs[0])?;
            if x0 != x1 {
                return Err("pairwise: the two halves read different inputs".into());
            }
            let rows = 2 * self.ty(w0).shape().rows();
            let (wl, wh) = (self.sliced(w0, 0, rows / 2, "weights")?, self.sliced(w1, rows / 2, rows, "weights")?);
            let (bl, bh) = (self.sliced(b0, 0, rows / 2, "bias")?, self.sliced(b1, rows / 2, rows, "bias")?);
            if wl != wh || bl != bh {
                return Err("pairwise: the two halves must be slices of one affine layer".into());
            }
            let (l0w, l0f) = self.table(wl)?;
            return Ok(FtHalf { l0w, l0f, l0b: bl, input: x0, act: B200_ACT_CRELU, pairwise: true, rows });
        }
        Err("a product of two nodes is only recognised as pairwise_mul of a crelu".into())
    }

    /// loss = ((sigmoid(out) + (-1 * targets)) * the same).reduce_sum_batch()
    /// (builder.rs:351-354 `squared_error`, value/builder.rs:142) -> (out, targets)
    fn loss(&self, loss: NodeId) -> Result<(NodeId, NodeId), String> {
        let sum = self.made(loss)?;
        if !sum.name.starts_with("ReduceSum<Batch") {
            return Err(format!("loss: expected a sum over the batch, found {}", sum.name));
        }
        let sq = self.made(sum.inputs[0])?;
        if sq.name != "Binary.Mul" || sq.inputs[0] != sq.inputs[1] {
            return Err("loss: only squared error is supported (entry weights and other losses are not)".into());
        }
        let diff = self.made(sq.inputs[0])?;
        if diff.name != "Binary.Add" {
            return Err("loss: expected `prediction - targets`".into());
        }
        for (pred, neg) in [(diff.inputs[0], diff.inputs[1]), (diff.inputs[1], diff.inputs[0])] {
            let (p, n) = (self.made(pred)?, self.made(neg)?);
            if p.name == "Sigmoid" && n.name == "Binary.Mul" {
                // -1.0 * targets: one operand is a broadcast constant, the other the dense input
                for t in &n.inputs {
                    let t = self.unbroadcast(*t)?;
                    if self.input(t).is_some() {
                        return Ok((p.inputs[0], t));
                    }
                }
            }
        }
        Err("loss: expected `output.sigmoid().squared_error(targets)`".into())
    }
}

/// `ft_block_rows` is a property of the input featuriser, not of the graph: 768 for `Chess768` and
/// `ChessBucketsMirrored`, 147 for `Ataxx147`, 0 when nothing is known (the gather kernels run then).
pub fn recognise(defn: &ModelDefinition, ft_block_rows: usize, max_batch: usize) -> Result<Recognised, String> {
    let w = Walk { ir: defn.ir() };
    let loss = defn.loss().ok_or("the model has no loss node")?;
    let (out, targets) = w.loss(loss)?;
    if defn.outputs().iter().all(|(id, _)| *id != out) {
        return Err("the loss is not taken on the registered model output".into());
    }

    // from the output downwards: [activation] [select] affine, until the concat
    struct Layer {
        w: NodeId,
        b: NodeId,
        act: i32,
    }
    let mut layers: Vec<Layer> = Vec::new();
    let mut buckets: Option<NodeId> = None;
    let mut node = out;
    loop {
        let mut m = w.made(node)?;
        if m.name == "Concat" {
            break;
        }
        if layers.len() == 3 {
            return Err("more than three dense layers".into());
        }
        let mut act = B200_ACT_NONE;
        match m.name.as_str() {
            "CReLU" => act = B200_ACT_CRELU,
            "SCReLU" => act = B200_ACT_SCRELU,
            _ => {}
        }
        if act != B200_ACT_NONE {
            node = m.inputs[0];
            m = w.made(node)?;
        }
        if m.name == "Select" {
            let idx = w.unbroadcast(m.inputs[1])?;
            if buckets.is_some_and(|b| b != idx) {
                return Err("dense layers select by different inputs".into());
            }
            buckets = Some(idx);
            node = m.inputs[0];
        }
        let (lw, lb, x) = w.affine(node)?;
        if w.weight(lw).is_none() || w.weight(lb).is_none() {
            return Err("dense layer: weights and bias must be plain weights".into());
        }
        layers.push(Layer { w: lw, b: lb, act });
        node = x;
    }
    if layers.is_empty() {
        return Err("no dense layer above the concat".into());
    }
    let concat = w.made(node)?;
    let (s, n) = (w.ft_half(concat.inputs[0])?, w.ft_half(concat.inputs[1])?);
    if (s.l0w, s.l0f, s.l0b, s.act, s.pairwise) != (n.l0w, n.l0f, n.l0b, n.act, n.pairwise) {
        return Err("the two perspectives must share one feature transformer".into());
    }
    if s.input == n.input {
        return Err("both halves of the concat read the same input".into());
    }
    let (sty, nty) = (w.ty(s.input), w.ty(n.input));
    let (Layout::Sparse(nnz), Layout::Sparse(nnz_n)) = (sty.layout(), nty.layout()) else {
        return Err("feature transformer: the inputs are not sparse".into());
    };
    if nnz != nnz_n || sty.shape().rows() != nty.shape().rows() {
        return Err("the perspective inputs differ in size".into());
    }

    let n_buckets = buckets.map_or(1, |b| w.ty(b).shape().rows());
    let mut desc = b200_net_desc {
        n_inputs: sty.shape().rows() as i32,
        nnz: nnz as i32,
        ft_out: s.rows as i32,
        ft_act: s.act,
        pairwise: s.pairwise as i32,
        factoriser_rows: s.l0f.map_or(0, |f| w.ty(f).shape().cols() as i32),
        n_out_buckets: n_buckets as i32,
        n_dense: layers.len() as i32,
        ft_block_rows: ft_block_rows as i32,
        max_batch: max_batch as i32,
        ..Default::default()
    };
    let name = |id: NodeId| w.weight(id).unwrap().to_string();
    let mut weights = vec![(name(s.l0w), "l0w"), (name(s.l0b), "l0b")];
    if let Some(f) = s.l0f {
        weights.push((name(f), "l0f"));
    }
    const DENSE: [(&str, &str); 3] = [("l1w", "l1b"), ("l2w", "l2b"), ("l3w", "l3b")];
    let mut fan_in = if s.pairwise { s.rows } else { 2 * s.rows };
    for (i, layer) in layers.iter().rev().enumerate() {
        let shape = w.ty(layer.w).shape();
        if shape.cols() != fan_in || shape.rows() % n_buckets != 0 {
            return Err(format!("dense layer {}: {}x{} does not fit {fan_in} inputs and {n_buckets} buckets", i + 1, shape.rows(), shape.cols()));
        }
        desc.dense_out[i] = (shape.rows() / n_buckets) as i32;
        desc.dense_act[i] = layer.act;
        fan_in = shape.rows() / n_buckets;
        weights.push((name(layer.w), DENSE[i].0));
        weights.push((name(layer.b), DENSE[i].1));
    }
    if desc.dense_out[layers.len() - 1] != 1 || desc.dense_act[layers.len() - 1] != B200_ACT_NONE {
        return Err("the network output must be one value per position, without an activation".into());
    }
    // every weight of the graph must have found its place: anything left over is a part of the
    // model this back end would silently ignore (examples/tests/test2.rs:50-65 is such a graph)
    let known: BTreeMap<&str, ()> = weights.iter().map(|(id, _)| (id.as_str(), ())).collect();
    for (_, (id, _)) in defn.ir().weights() {
        if !known.contains_key(id.as_str()) {
            return Err(format!("weight '{id}' is not part of the recognised network"));
        }
    }
    let input_name = |id: NodeId| w.input(id).map(str::to_string).ok_or("a network input is not a registered model input");
    Ok(Recognised {
        desc,
        weights,
        stm: input_name(s.input)?,
        ntm: input_name(n.input)?,
        buckets: buckets.map(input_name).transpose()?,
        targets: input_name(targets)?,
    })
}
