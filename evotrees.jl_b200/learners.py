"""Learner configurations mirroring the reference's keyword constructors (src/learners.jl).

Only the hyper-parameters that reach the device path are kept; names, defaults and validation follow
`EvoTreeRegressor` (src/learners.jl:25-119), `EvoTreeClassifier` and `EvoTreeMLE` (min_weight defaults
to 8 there) and `check_args` (src/learners.jl:522-552).
"""
from __future__ import annotations

from dataclasses import dataclass, field

_REG_LOSSES = ("mse", "logloss", "poisson", "gamma", "tweedie", "mae", "cred_var", "cred_std", "quantile", "multiquantile")
_MLE_LOSSES = ("gaussian_mle", "logistic_mle")


def _check(name, value, lo, hi):
    if not (lo <= value <= hi):
        raise ValueError(f"Invalid value for parameter `{name}`: {value}. `{name}` must be between {lo} and {hi}.")


@dataclass
class EvoTypes:
    loss: str = "mse"
    nrounds: int = 100
    bagging_size: int = 1
    L2: float = 1.0
    lambda_: float = 0.0
    gamma: float = 0.0
    eta: float = 0.1
    max_depth: int = 6
    min_weight: float = 1.0
    rowsample: float = 1.0
    colsample: float = 1.0
    nbins: int = 64
    monotone_constraints: dict = field(default_factory=dict)  # {feature (1-based): -1 | 0 | 1}
    tree_type: str = "binary"
    seed: int = 123
    device: str = "gpu"
    early_stopping_rounds: int = 2 ** 62
    early_stopping_tolerance: float = 0.0
    alpha: float = 0.5          # quantile loss / metric
    alphas: tuple = (0.1, 0.5, 0.9)   # multiquantile loss / metric (src/learners.jl:45)
    metric: str | None = None

    _losses = ()
    _metrics = ()

    def __post_init__(self):
        self.loss = str(self.loss)
        if self.loss == "linear":
            self.loss = "mse"
        if self.loss == "logistic":   # EvoTreeMLE: :logistic_mle; EvoTreeRegressor: the old name of :logloss
            self.loss = "logistic_mle" if "logistic_mle" in self._losses else "logloss"
        if self.loss == "gaussian":
            self.loss = "gaussian_mle"
        if self.loss not in self._losses:
            raise ValueError(f"Invalid loss. Must be one of: {list(self._losses)}")
        # metric defaults to the loss (src/learners.jl:75-87, 260, 352-365)
        default_metric = "mae" if self.loss in ("cred_var", "cred_std") else self.loss   # src/learners.jl:76-80
        self.metric = default_metric if self.metric is None else str(self.metric)
        if self.metric == "gaussian":
            self.metric = "gaussian_mle"
        if self.metric == "logistic":
            self.metric = "logistic_mle"
        if self.metric not in self._metrics:
            raise ValueError(f"Invalid metric. Must be one of: {list(self._metrics)}")
        self.check_args()

    def check_args(self):
        _check("nrounds", self.nrounds, 0, 2 ** 62)
        _check("max_depth", self.max_depth, 1, 15)
        _check("nbins", self.nbins, 2, 255)
        _check("lambda", self.lambda_, 0.0, float("inf"))
        _check("gamma", self.gamma, 0.0, float("inf"))
        _check("min_weight", self.min_weight, 0.0, float("inf"))
        _check("rowsample", self.rowsample, 2.220446049250313e-16, 1.0)
        _check("colsample", self.colsample, 2.220446049250313e-16, 1.0)
        _check("eta", self.eta, 0.0, float("inf"))
        _check("bagging_size", self.bagging_size, 1, 2 ** 31)
        _check("early_stopping_tolerance", self.early_stopping_tolerance, 0.0, float("inf"))
        _check("alpha", self.alpha, 0.0, 1.0)
        if self.loss == "multiquantile":       # check_alphas, src/learners.jl:505-520
            self.alphas = tuple(float(a) for a in self.alphas)
            if not 1 <= len(self.alphas) <= 8 or any(not 0.0 < a < 1.0 for a in self.alphas):
                raise ValueError("`alphas` must hold 1 to 8 values strictly between 0 and 1")
        self.tree_type = str(self.tree_type).lstrip(":")
        if self.tree_type not in ("binary", "oblivious"):   # src/learners.jl: tree_type ∈ (:binary, :oblivious)
            raise ValueError("Invalid input for `tree_type` parameter: must be `binary` or `oblivious`")
        if self.device not in ("gpu", "cuda"):
            raise ValueError("device must be :gpu / :cuda: this package has no CPU path")


@dataclass
class EvoTreeRegressor(EvoTypes):
    _losses = _REG_LOSSES
    _metrics = ("mse", "rmse", "mae", "logloss", "poisson", "gamma", "tweedie", "quantile", "multiquantile")


@dataclass
class EvoTreeClassifier(EvoTypes):
    loss: str = "mlogloss"
    _losses = ("mlogloss",)
    _metrics = ("mlogloss",)


@dataclass
class EvoTreeMLE(EvoTypes):
    loss: str = "gaussian_mle"
    min_weight: float = 8.0
    _losses = _MLE_LOSSES
    _metrics = ("gaussian_mle", "logistic_mle")


@dataclass
class EvoTreeCount(EvoTypes):
    """`EvoTreeCount` (src/learners.jl:122-200): poisson loss and metric."""
    loss: str = "poisson"
    _losses = ("poisson",)
    _metrics = ("poisson",)
