"""The residual stream of a step: the float32 running sum x [T, dim] plus,
possibly, something that is still owed to it.

A product whose sum over K was split across blocks leaves its result as a few
partial sums.  Instead of a kernel that only adds them up, the stream keeps
them `pending` and the next kernel that reads x completes the sum on its way:
RMSNorm does (it reads every element of x anyway), so split reduction, residual
add and norm are one pass.  In the same way a block that norms a sublayer's
output before it adds it (`add_normed`) leaves that sum to the next norm that
reads x, which then does both norms in one pass over the row.  Parts use

    residual.add_linear(a, w)        x += a @ w.T   (fused into the product's epilogue, or deferred)
    residual.add(y)                  x += y         (for parts that cannot fuse)
    residual.add_normed(y, norm, m)  x += m * norm(y), y a `Branch`  (deferred to the next norm, or resolved)
    residual.add_scaled(y, s)        x += s * y, y a `Branch`, s a per-column factor [dim]  (deferred the same way)
    residual.tensor()                x, complete

`Branch` is a stream of its own that starts empty: what a sublayer "adds" to it
is its output, kept in 32-bit (or as the partial sums of its last product).
"""
import torch

from .. import ops


class Residual:
    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending = None
        self.normed = None                 # (Branch, norm part, factor) still to be added
        self.scaled = []                   # (Branch, per-column factor) still to be added

    def resolve(self) -> None:
        if self.scaled:
            owed, self.scaled = self.scaled, []
            for i in range(0, len(owed), 2):
                ops.layernorm_multi(self.x, [(b.value(), s) for b, s in owed[i:i + 2]])
        if self.normed is not None:
            branch, norm, mult = self.take_normed()
            norm.add_into(self.x, branch, mult)
        if self.pending is not None:
            ops.add_partials(self.x, self.pending)
            self.pending = None

    def tensor(self) -> torch.Tensor:
        self.resolve()
        return self.x

    def add_linear(self, a, w) -> None:
        self.resolve()
        self.pending = ops.linear(a, w, self.x, mode="add", defer=True)

    def add(self, y) -> None:
        self.resolve()
        ops.add_into(self.x, y)

    def add_normed(self, branch: "Branch", norm, mult: float) -> None:
        self.resolve()
        self.normed = (branch, norm, float(mult))

    def add_scaled(self, branch: "Branch", scale) -> None:
        """x += scale * branch (scale: a vector over the columns).  Left to the next norm that reads x."""
        if self.normed is not None or self.pending is not None:
            self.resolve()
        self.scaled.append((branch, scale))

    def take_scaled(self):
        s, self.scaled = self.scaled, []
        return s

    def take_normed(self):
        n, self.normed = self.normed, None
        return n

    def take_pending(self):
        """The partial sums still owed to x (the caller adds them); a normed or scaled branch is added first."""
        if self.scaled:
            owed, self.scaled = self.scaled, []
            for i in range(0, len(owed), 2):
                ops.layernorm_multi(self.x, [(b.value(), s) for b, s in owed[i:i + 2]])
        if self.normed is not None:
            branch, norm, mult = self.take_normed()
            norm.add_into(self.x, branch, mult)
        p, self.pending = self.pending, None
        return p


class Branch(Residual):
    """The output of one sublayer on its way into a stream: float32 [T, dim], empty at first, so the first
    product "added" to it is stored, or left as the partial sums of a split over K (`partials`, x unwritten)."""

    def __init__(self, n_tokens: int, dim: int, device):
        super().__init__(torch.empty(n_tokens, dim, dtype=torch.float32, device=device))
        self.empty = True
        self.partials = None

    def _materialise(self) -> None:
        if self.empty:
            self.x.zero_()
            self.empty = False
        if self.partials is not None:
            p, self.partials = self.partials, None
            self.x.zero_()
            ops.add_partials(self.x, p)

    def add_linear(self, a, w) -> None:
        if self.empty:
            self.partials = ops.linear(a, w, self.x, mode="store", defer=True)
            self.empty = False
            return
        self._materialise()
        super().add_linear(a, w)

    def add(self, y) -> None:
        self._materialise()
        super().add(y)

    def resolve(self) -> None:
        self._materialise()
        super().resolve()

    def value(self) -> torch.Tensor:
        """The branch as the norm kernels take it: the complete float32 [T, dim] tensor, or partial sums [S, T, dim]."""
        if self.partials is not None and self.pending is None and self.normed is None and not self.scaled:
            p, self.partials = self.partials, None
            self.empty = True
            return p
        return self.tensor()


def as_residual(x) -> "Residual":
    return x if isinstance(x, Residual) else Residual(x)
