"""Kernel registry: public names resolved from literal ``KERNEL_META`` declarations.

Behavioural mirror of tirx_kernels/registry.py in the reference (index :173-216,
load_kernel :253-267, discover_kernels :278-299, CLI :302-329): the index is derived from
source text, so looking up one kernel imports exactly one module; a module's runtime
``KERNEL_META`` must agree with the indexed one; duplicate public names are an error;
``bench``, ``test``, ``bench_suite``, ``experimental`` and any ``utils`` subpackage are not
kernel buckets.
"""

from __future__ import annotations

import ast
import importlib
import logging
import re
from dataclasses import dataclass
from pathlib import Path
from types import ModuleType

import tirx_kernels

_log = logging.getLogger(__name__)

NON_CATEGORY_DIRS = frozenset({"bench", "test", "bench_suite", "experimental"})
HELPER_SUBPACKAGES = frozenset({"utils"})
_META_FIELDS = (("name", str), ("category", str), ("compute_capability", int))
_ASSIGN_RE = re.compile(r"^KERNEL_META\s*=", re.MULTILINE)


@dataclass(frozen=True)
class KernelRecord:
    name: str
    category: str
    compute_capability: int
    module_name: str
    source_path: Path


def _package_root() -> Path:
    return Path(tirx_kernels.__file__).resolve().parent


def discover_categories() -> list[str]:
    names = []
    for entry in sorted(_package_root().iterdir()):
        if not entry.is_dir() or entry.name.startswith("_") or entry.name in NON_CATEGORY_DIRS:
            continue
        if (entry / "__init__.py").is_file():
            names.append(entry.name)
    return names


def _walk_modules(directory: Path, prefix: str = ""):
    """Yield (dotted name relative to the category, path) for every candidate module."""
    for entry in sorted(directory.iterdir()):
        if entry.name.startswith("_"):
            continue
        if entry.is_file() and entry.suffix == ".py":
            yield prefix + entry.stem, entry
        elif entry.is_dir() and entry.name not in HELPER_SUBPACKAGES and (entry / "__init__.py").is_file():
            yield from _walk_modules(entry, f"{prefix}{entry.name}.")


def _meta_problems(meta, category: str) -> list[str]:
    if not isinstance(meta, dict):
        return [f"expected dict, got {type(meta).__name__}"]
    problems = []
    for key, kind in _META_FIELDS:
        value = meta.get(key)
        if isinstance(value, bool) or not isinstance(value, kind):
            problems.append(f"{key!r} must be {kind.__name__}")
        elif kind is str and not value:
            problems.append(f"{key!r} must not be empty")
    if meta.get("category") != category:
        problems.append(f"'category' is {meta.get('category')!r}, expected containing category {category!r}")
    return problems


def _read_literal_meta(path: Path) -> dict | None:
    """The dict literal assigned to a module-level ``KERNEL_META``, or None when absent."""
    text = path.read_text(encoding="utf-8")
    if not _ASSIGN_RE.search(text):
        return None
    found = []
    for node in ast.parse(text, filename=str(path)).body:
        targets = []
        if isinstance(node, ast.Assign):
            targets = node.targets
        elif isinstance(node, ast.AnnAssign) and node.value is not None:
            targets = [node.target]
        if any(isinstance(t, ast.Name) and t.id == "KERNEL_META" for t in targets):
            value = ast.literal_eval(node.value)
            if not isinstance(value, dict):
                raise ValueError(f"{path} KERNEL_META must be a literal dict")
            found.append(value)
    if len(found) > 1:
        raise ValueError(f"{path} assigns KERNEL_META more than once")
    return found[0] if found else None


_INDEX_CACHE: dict = {"stamp": None, "records": {}, "diagnostics": ()}


def _scan() -> tuple[tuple, list[tuple[str, str, Path]]]:
    candidates = []
    stamp = []
    for category in discover_categories():
        for relative, path in _walk_modules(_package_root() / category):
            info = path.stat()
            candidates.append((category, relative, path))
            stamp.append((str(path), info.st_mtime_ns, info.st_size))
    return tuple(stamp), candidates


def kernel_index(*, strict: bool = False) -> dict[str, KernelRecord]:
    """Public name -> record, rebuilt only when a candidate source file changes."""
    stamp, candidates = _scan()
    if _INDEX_CACHE["stamp"] != stamp:
        records: dict[str, KernelRecord] = {}
        diagnostics = []
        for category, relative, path in candidates:
            module_name = f"tirx_kernels.{category}.{relative}"
            try:
                meta = _read_literal_meta(path)
            except (SyntaxError, ValueError) as error:
                diagnostics.append(f"{path} has invalid KERNEL_META: {error}")
                continue
            if meta is None:
                continue
            problems = _meta_problems(meta, category)
            if problems:
                diagnostics.append(f"{module_name} has invalid KERNEL_META: " + "; ".join(problems))
                continue
            if meta["name"] in records:
                raise ValueError(
                    f"duplicate kernel registry name {meta['name']!r}: "
                    f"{records[meta['name']].module_name} and {module_name}"
                )
            records[meta["name"]] = KernelRecord(meta["name"], category, meta["compute_capability"],
                                                 module_name, path)
        _INDEX_CACHE.update(stamp=stamp, records=records, diagnostics=tuple(diagnostics))
    if _INDEX_CACHE["diagnostics"]:
        if strict:
            raise ValueError(_INDEX_CACHE["diagnostics"][0])
        for message in _INDEX_CACHE["diagnostics"]:
            _log.warning(message)
    return dict(_INDEX_CACHE["records"])


def _import_checked(record: KernelRecord, *, strict: bool) -> ModuleType | None:
    try:
        module = importlib.import_module(record.module_name)
    except Exception as error:
        if strict:
            raise
        _log.warning("tirx_kernels: failed to import %s: %s", record.module_name, error)
        return None
    meta = getattr(module, "KERNEL_META", None)
    problems = _meta_problems(meta, record.category)
    if isinstance(meta, dict):
        if meta.get("name") != record.name:
            problems.append(f"runtime name {meta.get('name')!r} does not match source index {record.name!r}")
        if meta.get("compute_capability") != record.compute_capability:
            problems.append("runtime compute_capability does not match source index")
    if problems:
        message = f"{record.module_name} has invalid runtime KERNEL_META: " + "; ".join(problems)
        if strict:
            raise ValueError(message)
        _log.warning(message)
        return None
    return module


def load_kernel(name: str, *, strict: bool = False) -> ModuleType:
    """Import the one module whose ``KERNEL_META['name']`` is `name`; KeyError if there is none."""
    record = kernel_index(strict=strict).get(name)
    module = _import_checked(record, strict=strict) if record is not None else None
    if module is None:
        raise KeyError(name)
    return module


def check_workload_imports(workloads: list[dict], *, strict: bool = True) -> list[str]:
    names = sorted({w["kernel"] for w in workloads})
    for name in names:
        load_kernel(name, strict=strict)
    return names


def discover_kernels(*, min_compute_capability: int | None = None, category: str | None = None,
                     strict: bool = False) -> dict[str, ModuleType]:
    """``{public_name: module}`` for every registered kernel passing the filters."""
    modules = {}
    for name, record in kernel_index(strict=strict).items():
        if category is not None and record.category != category:
            continue
        if min_compute_capability is not None and record.compute_capability != min_compute_capability:
            continue
        module = _import_checked(record, strict=strict)
        if module is not None:
            modules[name] = module
    return modules


def _main() -> None:
    import argparse
    import json

    parser = argparse.ArgumentParser(description="List registered kernels")
    parser.add_argument("--list", action="store_true", help="List all kernels")
    parser.add_argument("--format", choices=["text", "json", "benchrun"], default="text")
    parser.add_argument("--category", type=str, default=None)
    parser.add_argument("--cc", type=int, default=None, help="Compute capability filter")
    parser.add_argument("--strict", action="store_true", help="Raise on the first import failure")
    args = parser.parse_args()
    kernels = discover_kernels(min_compute_capability=args.cc, category=args.category, strict=args.strict)
    if args.format == "json":
        print(json.dumps(
            [{"name": n, "meta": m.KERNEL_META, "configs": getattr(m, "CONFIGS", [])}
             for n, m in sorted(kernels.items())], indent=2))
    elif args.format == "benchrun":
        for name, module in sorted(kernels.items()):
            for config in getattr(module, "CONFIGS", []):
                label = config.get("label", "default")
                print(f"{name}|{label}|python -m tirx_kernels.bench --kernel {name} "
                      f"--config {label} --json-file {{json_file}}")
    else:
        for name, module in sorted(kernels.items()):
            meta = module.KERNEL_META
            print(f"  {name:30s}  {meta.get('category', '?'):12s}  "
                  f"sm{meta.get('compute_capability', 0) * 10}  ({len(getattr(module, 'CONFIGS', []))} configs)")


if __name__ == "__main__":
    _main()
