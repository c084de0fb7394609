"""`triton-ext.conf` metadata and TRITON_EXT_NAMES gating.

Follows the reference's CMake helpers: the file holds one semicolon-separated line
``name;status[;hash]`` (cmake/utils.cmake:94-122, default status "experimental" at :96); an extension
is built when TRITON_EXT_NAMES is empty or lists its name (cmake/utils.cmake:73-84). The reference's
code reads ``triton-ext.conf`` (cmake/utils.cmake:53,94) while its README speaks of
``triton_ext.conf`` (README.md:137); both spellings are accepted here, the hyphen first.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Iterable, Optional

CONF_NAMES = ("triton-ext.conf", "triton_ext.conf")


@dataclass(frozen=True)
class ExtConf:
    name: str
    status: str = "experimental"
    hash: str = ""
    path: str = ""


def parse_conf_text(text: str, path: str = "") -> ExtConf:
    """Parse ``name;status[;hash]``. Raises ValueError when the name is missing
    (the reference stops the configure step with FATAL_ERROR, cmake/utils.cmake:124-126)."""
    parts = [p.strip() for p in text.strip().split(";")] if text.strip() else []
    if not parts or not parts[0]:
        raise ValueError(f"triton-ext.conf not found or empty: {path or '<text>'}")
    status = parts[1] if len(parts) >= 2 and parts[1] else "experimental"
    hash_ = parts[2] if len(parts) >= 3 else ""
    return ExtConf(parts[0], status, hash_, path)


def find_conf(ext_dir: str) -> Optional[str]:
    for name in CONF_NAMES:
        p = os.path.join(ext_dir, name)
        if os.path.exists(p):
            return p
    return None


def read_conf(ext_dir: str) -> ExtConf:
    p = find_conf(ext_dir)
    if p is None:
        raise ValueError(f"triton-ext.conf not found or empty in {ext_dir}")
    with open(p) as f:
        return parse_conf_text(f.read(), p)


def ext_names_filter(value: Optional[str] = None) -> list[str]:
    """The TRITON_EXT_NAMES allow-list (a CMake list: semicolon separated; commas tolerated)."""
    if value is None:
        value = os.environ.get("TRITON_EXT_NAMES", "")
    return [v.strip() for v in value.replace(",", ";").split(";") if v.strip()]


def should_build(ext_dir: str, names: Optional[Iterable[str]] = None) -> bool:
    """True when the directory has a conf with a name and the allow-list is empty or holds it
    (triton_ext_should_build_extension, cmake/utils.cmake:52-87)."""
    p = find_conf(ext_dir)
    if p is None:
        return False
    with open(p) as f:
        text = f.read().strip()
    if not text:
        return False
    name = text.split(";")[0].strip()
    allow = list(names) if names is not None else ext_names_filter()
    return True if not allow else name in allow


def discover(root: str) -> list[ExtConf]:
    """Every sub-directory of `root` that carries a conf (pass/CMakeLists.txt:6-18 does the same
    glob over pass/*)."""
    out = []
    if not os.path.isdir(root):
        return out
    for entry in sorted(os.listdir(root)):
        d = os.path.join(root, entry)
        if os.path.isdir(d) and find_conf(d):
            out.append(read_conf(d))
    return out
