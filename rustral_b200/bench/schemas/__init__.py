"""The JSON Schema files of the benchmark and manifest documents, and a validator for the subset of JSON Schema they use
(type, const, enum, required, properties, items, minItems, pattern), so that checking a document needs no third-party
package (the reference validates with scripts/bench/validate_schema.py against benchmarks/schema_v2.json)."""
from __future__ import annotations

import json
import re
from pathlib import Path

_DIR = Path(__file__).resolve().parent
NAMES = ("schema_v2", "manifest_schema", "curated_manifest_schema")


def load(name: str) -> dict:
    if name not in NAMES:
        raise KeyError(f"unknown schema {name!r}; known: {NAMES}")
    return json.loads((_DIR / f"{name}.json").read_text())


_TYPES = {"object": dict, "array": list, "string": str, "boolean": bool, "null": type(None)}


def _is(value, tname: str) -> bool:
    if tname == "number":
        return isinstance(value, (int, float)) and not isinstance(value, bool)
    if tname == "integer":
        return isinstance(value, int) and not isinstance(value, bool)
    return isinstance(value, _TYPES[tname])


def validate(value, schema: dict, where: str = "$") -> list:
    """Problems of `value` against `schema` (empty list: valid)."""
    errs = []
    if "const" in schema and value != schema["const"]:
        errs.append(f"{where}: must be {schema['const']!r}, is {value!r}")
    if "enum" in schema and value not in schema["enum"]:
        errs.append(f"{where}: {value!r} is not one of {schema['enum']}")
    t = schema.get("type")
    if t is not None:
        names = t if isinstance(t, list) else [t]
        if not any(_is(value, n) for n in names):
            errs.append(f"{where}: expected {' or '.join(names)}, got {type(value).__name__}")
            return errs
    if isinstance(value, str) and "pattern" in schema and not re.search(schema["pattern"], value):
        errs.append(f"{where}: {value!r} does not match {schema['pattern']}")
    if isinstance(value, dict):
        for k in schema.get("required", []):
            if k not in value:
                errs.append(f"{where}: missing key {k!r}")
        for k, sub in schema.get("properties", {}).items():
            if k in value:
                errs += validate(value[k], sub, f"{where}.{k}")
    if isinstance(value, list):
        if len(value) < schema.get("minItems", 0):
            errs.append(f"{where}: needs at least {schema['minItems']} item(s)")
        if "items" in schema:
            for i, v in enumerate(value):
                errs += validate(v, schema["items"], f"{where}[{i}]")
    return errs


def check(doc, name: str) -> list:
    return validate(doc, load(name))
