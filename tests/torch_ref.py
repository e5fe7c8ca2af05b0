"""Independent PyTorch (CPU, float64, autograd) model of the training step.

Used only to validate the CPU oracle's hand-written backward pass: the forward is written
with dense one-hot style gathers and the gradients come from torch.autograd, so nothing is
shared with oracle/oracle.c beyond the network definition.
"""
import torch


def _act(kind, x):
    if kind == 0:
        return x
    c = x.clamp(0.0, 1.0)
    return c * c if kind == 2 else c


def net_loss(desc, tensors, stm, nstm, buckets, targets):
    """tensors: dict name -> torch float64 leaf (flat, column-major).  Returns (loss_sum, outputs)."""
    H, NI = desc.ft_out, desc.n_inputs
    W = tensors["l0w"].view(NI, H)
    if desc.factoriser_rows:
        W = W + tensors["l0f"].view(desc.factoriser_rows, H).repeat(NI // desc.factoriser_rows, 1)
    Wz = torch.cat([W, torch.zeros(1, H, dtype=W.dtype)], 0)  # row NI = "no feature"

    def ft(idx):
        idx = torch.as_tensor(idx, dtype=torch.long)
        idx = torch.where((idx >= 0) & (idx < NI), idx, torch.full_like(idx, NI))
        acc = Wz[idx].sum(1) + tensors["l0b"]
        if desc.pairwise:
            u = acc.clamp(0.0, 1.0)
            return u[:, : H // 2] * u[:, H // 2:]
        return _act(desc.ft_act, acc)

    x = torch.cat([ft(stm), ft(nstm)], 1)
    k = torch.as_tensor(buckets, dtype=torch.long)
    O = desc.n_out_buckets
    for l in range(desc.n_dense):
        M, K = desc.dense_out[l], desc.dense_in(l)
        Wl = tensors[f"l{l + 1}w"].view(K, O * M)          # column-major (O*M) x K
        z = x @ Wl + tensors[f"l{l + 1}b"]                  # all buckets
        z = z.view(-1, O, M)[torch.arange(len(k)), k]       # select
        x = _act(desc.dense_act[l], z)
    out = x[:, 0]
    s = torch.sigmoid(out)
    t = torch.as_tensor(targets, dtype=torch.float64)
    return ((s - t) ** 2).sum(), out


def grads(desc, tensors_np, stm, nstm, buckets, targets):
    leaves = {k: torch.tensor(v, dtype=torch.float64, requires_grad=True) for k, v in tensors_np.items()}
    loss, out = net_loss(desc, leaves, stm, nstm, buckets, targets)
    loss.backward()
    return float(loss.detach()), {k: v.grad.numpy() for k, v in leaves.items()}, out.detach().numpy()
