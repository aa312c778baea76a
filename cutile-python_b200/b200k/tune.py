"""Kernel-form tuning for the GEMM entry points.

The reference chooses tile sizes and CTA counts per shape with a measuring search
(`exhaustive_search`, src/cuda/tile/tune/_tune.py:132-336, returning a `TuningResult` of
`Measurement`s) and its benches carry the winners as constants.  The library here has a
fixed set of hand-written kernel forms instead of a compiler, so what there is to choose is
small: one-CTA or CTA-pair kernel, tile width, epilogue store form and the number of K
slices (`b200k_gemm_config` in include/b200k.h).  This module is the host side of that
choice:

* `GemmConfig` - one point of the search space;
* `use_config(cfg)` - a context in which every GEMM call of this thread uses `cfg`;
* `exhaustive_search(space, stream, run_fn)` - measure every config, drop the ones that can
  no longer win, return a `TuningResult`;
* `TuneDB` - winners per problem key in a JSON file; `set_db()` makes the GEMM wrappers
  look their shapes up (the `B200K_TUNE_DB` environment variable does the same at import);
* `tune_matmul`, `tune_block_scaled_matmul` - search for one concrete problem through the
  public wrappers and record the winner.
"""
from __future__ import annotations

import contextlib
import json
import math
import os
import threading
from dataclasses import asdict, dataclass
from typing import Any, Callable, Generic, Iterable, Sequence, TypeVar

import torch

from . import _lib

T = TypeVar("T")

KERNEL_AUTO, KERNEL_ONE_CTA, KERNEL_PAIR = 0, 1, 2
STORE_AUTO, STORE_DIRECT, STORE_STAGED = 0, 1, 2


@dataclass(frozen=True)
class GemmConfig:
    """One kernel form; 0 in a field leaves that choice to the library's heuristics."""
    kernel: int = 0           # 1 = one-CTA (128-row tiles), 2 = CTA pair (256-row tiles)
    tile_n: int = 0           # 128 | 256 (CTA-pair kernel, unscaled operands)
    epilogue_store: int = 0   # 1 = from registers, 2 = staged through shared memory
    split_k: int = 0          # 1 = never, n > 1 = up to n K slices (dense GEMM only)

    def __post_init__(self):
        if self.kernel not in (0, 1, 2):
            raise ValueError(f"kernel must be 0, 1 or 2 (got {self.kernel})")
        if self.tile_n not in (0, 128, 256):
            raise ValueError(f"tile_n must be 0, 128 or 256 (got {self.tile_n})")
        if self.epilogue_store not in (0, 1, 2):
            raise ValueError(f"epilogue_store must be 0, 1 or 2 (got {self.epilogue_store})")
        if self.split_k < 0:
            raise ValueError(f"split_k must be >= 0 (got {self.split_k})")

    def to_c(self) -> "_lib.GemmConfig":
        return _lib.GemmConfig(self.kernel, self.tile_n, self.epilogue_store, self.split_k)

    @staticmethod
    def from_dict(d: dict) -> "GemmConfig":
        return GemmConfig(**{k: int(d.get(k, 0)) for k in ("kernel", "tile_n", "epilogue_store", "split_k")})


AUTO = GemmConfig()

# ---- the config a GEMM call uses ----------------------------------------------------------
_tls = threading.local()
_db: "TuneDB | None" = None


@contextlib.contextmanager
def use_config(cfg: GemmConfig | None):
    """Every GEMM this thread issues inside the block uses `cfg` (None: back to automatic,
    ignoring the database)."""
    prev = getattr(_tls, "override", None)
    _tls.override = (cfg if cfg is not None else AUTO,)
    try:
        yield
    finally:
        _tls.override = prev


def set_db(db: "TuneDB | str | None") -> None:
    """Install the database the GEMM wrappers consult (a TuneDB, a path, or None)."""
    global _db
    _db = TuneDB.load(db) if isinstance(db, (str, os.PathLike)) else db


def get_db() -> "TuneDB | None":
    return _db


def gemm_key(op: str, ab_dtype: int, c_dtype: int, layout: int, m: int, n: int, k: int, batch: int) -> str:
    """Problem key: operation, operand/output dtype enums, B layout and the four extents."""
    return f"{op}:{ab_dtype}:{c_dtype}:{layout}:{m}x{n}x{k}x{batch}"


def config_for(op: str, ab_dtype: int, c_dtype: int, layout: int, m: int, n: int, k: int,
               batch: int) -> GemmConfig | None:
    """The config for the GEMM call being issued: this thread's override, else the database
    entry of the problem, else None (automatic).  Costs nothing when neither is in use."""
    override = getattr(_tls, "override", None)
    if override is None and _db is None:
        return None
    key = gemm_key(op, ab_dtype, c_dtype, layout, m, n, k, batch)
    _tls.last_key = key
    if override is not None:
        return None if override[0] == AUTO else override[0]
    return _db.get(key)


def in_use() -> bool:
    """True while this thread runs under an override or a database is installed: the GEMM
    wrappers then look a config up per call instead of replaying a remembered launch."""
    return _db is not None or getattr(_tls, "override", None) is not None


def last_key() -> str | None:
    """Key of the last GEMM this thread issued under an override or with a database."""
    return getattr(_tls, "last_key", None)


# ---- database ----------------------------------------------------------------------------
class TuneDB:
    """Winning configs per problem key, kept as JSON: {"device": ..., "entries": {key:
    {"config": {...}, "mean_us": ...}}}."""

    def __init__(self, device: str = ""):
        self.device = device
        self.entries: dict[str, dict] = {}

    def get(self, key: str) -> GemmConfig | None:
        e = self.entries.get(key)
        return GemmConfig.from_dict(e["config"]) if e is not None else None

    def put(self, key: str, cfg: GemmConfig, mean_us: float | None = None) -> None:
        self.entries[key] = {"config": asdict(cfg), "mean_us": mean_us}

    def save(self, path) -> None:
        tmp = f"{path}.tmp"
        with open(tmp, "w") as f:
            json.dump({"device": self.device, "entries": self.entries}, f, indent=1, sort_keys=True)
        os.replace(tmp, path)

    @staticmethod
    def load(path) -> "TuneDB":
        with open(path) as f:
            d = json.load(f)
        db = TuneDB(d.get("device", ""))
        for key, e in d.get("entries", {}).items():
            GemmConfig.from_dict(e["config"])   # validates
            db.entries[key] = e
        return db

    def __len__(self):
        return len(self.entries)


# ---- measuring search --------------------------------------------------------------------
@dataclass(frozen=True)
class Measurement(Generic[T]):
    config: T
    mean_us: float
    num_samples: int
    error_margin_us: float    # half of the 95 % confidence interval of the mean


@dataclass(frozen=True)
class TuningResult(Generic[T]):
    best: Measurement
    successes: Sequence[Measurement]
    failures: Sequence[tuple]          # (config, exception type, message)

    def summary(self, top_k: int = 10) -> str:
        rows = sorted(self.successes, key=lambda m: m.mean_us)[:top_k]
        lines = [f"{len(self.successes)} configs measured, {len(self.failures)} failed"]
        lines += [f"  {m.mean_us:10.2f} us +- {m.error_margin_us:6.2f} ({m.num_samples:4d} samples)  {m.config}"
                  for m in rows]
        lines.append(f"best: {self.best.config} ({self.best.mean_us:.2f} us)")
        return "\n".join(lines)

    def __str__(self):
        return self.summary()


@dataclass
class _Running:
    config: Any
    order: int
    n: int = 0
    mean: float = 0.0
    m2: float = 0.0

    def add(self, us: float) -> None:
        self.n += 1
        d = us - self.mean
        self.mean += d / self.n
        self.m2 += d * (us - self.mean)

    @property
    def margin(self) -> float:
        if self.n < 2:
            return math.inf
        return 1.96 * math.sqrt(self.m2 / (self.n - 1) / self.n)

    def settled(self, max_samples: int, budget_us: float) -> bool:
        return self.n >= 5 and (self.margin <= 0.01 * self.mean or self.margin <= 0.5
                                or self.n >= max_samples or self.mean * self.n > budget_us)


class _EventTimer:
    """One sample = L2 flush, start event, run_fn(config), end event, on `stream`.  The flush
    (a zero fill four times the L2) also keeps the GPU busy while the host enqueues the call,
    so that short kernels are timed on the device and not by their launch path."""

    def __init__(self, stream, flush_bytes: int = 512 << 20):
        self.stream = stream if stream is not None else torch.cuda.current_stream()
        self.flush = torch.empty(flush_bytes, dtype=torch.uint8, device=self.stream.device) if flush_bytes else None
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)

    def __call__(self, run_fn, cfg) -> float:
        with torch.cuda.stream(self.stream):
            if self.flush is not None:
                self.flush.zero_()
            self.e0.record(self.stream)
            run_fn(cfg)
            self.e1.record(self.stream)
        self.e1.synchronize()
        return self.e0.elapsed_time(self.e1) * 1e3


def exhaustive_search(search_space: Sequence[T], stream, run_fn: Callable[[T], Any], *, quiet: bool = True,
                      warmup: int = 3, batch: int = 5, max_samples: int = 200,
                      budget_us_per_config: float = 2e6, timer: Callable | None = None,
                      validate: Callable[[T], None] | None = None) -> TuningResult[T]:
    """Measure `run_fn(config)` for every config of `search_space` and return the fastest.

    `run_fn` enqueues the work on the current stream.  Every config gets `warmup` untimed
    calls and a first batch of samples; after that, rounds of `batch` samples go to the
    configs that are neither settled (95 % interval within 1 % of the mean or 0.5 us, or out
    of samples/time) nor beaten (their interval lies wholly above the current best's).  A
    config whose call raises is recorded under `failures` and skipped.  `validate(config)`, if
    given, runs after a config's warm-up calls and raises when the config must not win (a
    wrong result, a device-side wait that gave up): time alone admits nobody.  `timer(run_fn,
    config) -> microseconds` replaces the CUDA-event timer (host-side tests)."""
    space = list(search_space)
    if not space:
        raise ValueError("Search space is empty.")
    if timer is None:
        timer = _EventTimer(stream)
    live: list[_Running] = []
    done: list[_Running] = []
    failures = []
    for i, cfg in enumerate(space):
        cand = _Running(cfg, i)
        try:
            for _ in range(warmup):
                run_fn(cfg)
            if validate is not None:
                validate(cfg)
            for _ in range(batch):
                cand.add(timer(run_fn, cfg))
        except Exception as e:  # noqa: BLE001 - a config the problem cannot take is data, not an error
            failures.append((cfg, type(e), str(e)))
            continue
        (done if cand.settled(max_samples, budget_us_per_config) else live).append(cand)

    while live:
        everyone = live + done
        leader = min(everyone, key=lambda c: (c.mean, c.order))
        bar = leader.mean + (leader.margin if math.isfinite(leader.margin) else 0.0)
        still = []
        for cand in live:
            if cand is not leader and cand.n >= 5 and cand.mean - cand.margin > bar:
                done.append(cand)          # cannot win any more
                continue
            try:
                for _ in range(batch):
                    cand.add(timer(run_fn, cand.config))
            except Exception as e:  # noqa: BLE001
                failures.append((cand.config, type(e), str(e)))
                continue
            (done if cand.settled(max_samples, budget_us_per_config) else still).append(cand)
        live = still

    if not done:
        cfg, exc, msg = failures[0]
        raise ValueError(f"No valid config found in search space.\nConfig: {cfg}\n{exc.__name__}: {msg}")
    successes = tuple(Measurement(c.config, c.mean, c.n, c.margin if math.isfinite(c.margin) else 0.0)
                      for c in sorted(done, key=lambda c: c.order))
    best = min(successes, key=lambda m: m.mean_us)
    result = TuningResult(best=best, successes=successes, failures=tuple(failures))
    if not quiet:
        print(result)
    return result


# ---- search spaces for the public wrappers -----------------------------------------------
def gemm_search_space(m: int, n: int, k: int, batch: int = 1, *, elem_bytes: int = 2,
                      block_scaled: bool = False, sms: int = 148) -> list[GemmConfig]:
    """Kernel forms worth measuring for one problem.  Always contains AUTO first, so the
    winner is never slower than the library's own choice (up to timing noise)."""
    space = [AUTO]
    for kernel in (KERNEL_PAIR, KERNEL_ONE_CTA):
        widths = (256, 128) if (kernel == KERNEL_PAIR and not block_scaled) else (0,)
        for tile_n in widths:
            for store in (STORE_DIRECT, STORE_STAGED):
                space.append(GemmConfig(kernel=kernel, tile_n=tile_n, epilogue_store=store, split_k=1))
    if not block_scaled:
        k_steps = -(-k * elem_bytes // 128)
        tiles = -(-m // 128) * -(-n // 256) * batch
        for split in (2, 3, 4, 6, 8, 12, 16, 24, 32):
            if split <= k_steps // 2 and tiles * split <= 2 * sms:
                space.append(GemmConfig(kernel=KERNEL_ONE_CTA, epilogue_store=STORE_STAGED, split_k=split))
    return space


def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


class _ResultGuard:
    """`validate` of the tune_* wrappers: a config may win only if, after its warm-up calls,
    the device status word is clean and the output equals the automatic form's (same product
    up to fp32 summation order).  A status word found set is cleared by the read, so it is
    not blamed on a later call."""

    def __init__(self, run, out: torch.Tensor, rtol: float = 2e-2):
        from . import _lib
        self._lib, self.run, self.out, self.rtol = _lib, run, out, rtol
        run(AUTO)
        torch.cuda.synchronize(out.device)
        code, info = _lib.device_status()
        if code != 0:
            raise _lib.B200KError(code, f"the automatic form tripped a device-side wait (info {info:#x})")
        self.want = out.float().clone()
        self.atol = rtol * float(self.want.abs().max()) if self.want.numel() else 0.0

    def __call__(self, cfg) -> None:
        self.out.zero_()
        self.run(cfg)
        torch.cuda.synchronize(self.out.device)
        code, info = self._lib.device_status()
        if code != 0:
            raise self._lib.B200KError(code, f"device-side wait gave up (info {info:#x})")
        torch.testing.assert_close(self.out.float(), self.want, rtol=self.rtol, atol=self.atol)


def tune_matmul(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor | None = None, *,
                db: TuneDB | None = None, search_space: Iterable[GemmConfig] | None = None,
                quiet: bool = True, **search_kw) -> TuningResult[GemmConfig]:
    """Search the kernel forms for `cutile_matmul(A, B, C)` / `bmm` (3-D operands) and record
    the winner in `db` (default: the installed database, if any)."""
    from . import matmul
    batched = A.dim() == 3
    m, k = A.shape[-2:]
    n = B.shape[-1]
    nb = A.shape[0] if batched else 1
    if C is None:
        C = torch.empty((*A.shape[:-1], n), dtype=A.dtype, device=A.device)
    space = list(search_space) if search_space is not None else gemm_search_space(
        m, n, k, nb, elem_bytes=A.element_size(), sms=_sm_count(A.device))

    def run(cfg):
        with use_config(cfg):
            matmul._gemm(A, B, C)

    search_kw.setdefault("validate", _ResultGuard(run, C))
    result = exhaustive_search(space, torch.cuda.current_stream(A.device), run, quiet=quiet, **search_kw)
    target = db if db is not None else _db
    if target is not None and last_key() is not None:
        target.put(last_key(), result.best.config, result.best.mean_us)
    return result


def tune_block_scaled_matmul(A, A_scale, B, B_scale, C=None, *, out_dtype=torch.float32,
                             db: TuneDB | None = None, search_space: Iterable[GemmConfig] | None = None,
                             quiet: bool = True, **search_kw) -> TuningResult[GemmConfig]:
    """Search the kernel forms for `cutile_block_scaled_matmul` on one MXFP8 problem."""
    from . import block_scaled
    m, k = A.shape
    n = B.shape[1]
    if C is None:
        C = torch.empty((m, n), dtype=out_dtype, device=A.device)
    space = list(search_space) if search_space is not None else gemm_search_space(
        m, n, k, 1, elem_bytes=1, block_scaled=True, sms=_sm_count(A.device))

    def run(cfg):
        with use_config(cfg):
            block_scaled.cutile_block_scaled_matmul(A, A_scale, B, B_scale, C=C)

    search_kw.setdefault("validate", _ResultGuard(run, C))
    result = exhaustive_search(space, torch.cuda.current_stream(A.device), run, quiet=quiet, **search_kw)
    target = db if db is not None else _db
    if target is not None and last_key() is not None:
        target.put(last_key(), result.best.config, result.best.mean_us)
    return result


if os.environ.get("B200K_TUNE_DB"):
    set_db(os.environ["B200K_TUNE_DB"])
