"""Error measure shared by the kernel numerics tests."""
import torch


def rel_err(a, b, row_tol=5e-2, abs_tol=3e-2):
    """Relative Frobenius error of ``a`` against the reference ``b``. Also asserts, so that one
    wrong row cannot hide in the norm of a large matrix: every row's relative error (row norms
    floored at a tenth of the mean row norm) stays under ``row_tol``, and the largest element
    error stays under ``abs_tol`` of the largest reference magnitude."""
    a, b = a.float(), b.float()
    d = a - b
    if b.dim() >= 2 and b.numel():
        d2, b2 = d.reshape(-1, b.shape[-1]), b.reshape(-1, b.shape[-1])
        rn = b2.norm(dim=1)
        row = d2.norm(dim=1) / torch.maximum(rn, 0.1 * rn.mean() + 1e-12)
        worst = int(row.argmax())
        assert row[worst].item() < row_tol, f"row {worst}: relative error {row[worst].item():.3e}"
    if b.numel():
        assert d.abs().max().item() <= abs_tol * b.abs().max().item() + 1e-6, \
            f"max abs error {d.abs().max().item():.3e} against max |ref| {b.abs().max().item():.3e}"
    return (d.norm() / (b.norm() + 1e-12)).item()
