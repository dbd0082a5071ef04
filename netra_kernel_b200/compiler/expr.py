"""Tiny integer expression language for launch shapes, constants and buffer sizes in the tactic
catalog and graph builders: names, integer literals, ``+ - * //``, parentheses and the functions
``ceil_div``, ``min``, ``max``, ``align``.  Evaluated over an explicit environment; nothing else
of Python is reachable."""
from __future__ import annotations

import ast
from typing import Mapping

from .types import ValidationError

_FUNCTIONS = {
    "ceil_div": lambda a, b: -(-a // b),
    "min": min,
    "max": max,
    "align": lambda a, b: -(-a // b) * b,
}
_BINARY = {ast.Add: lambda a, b: a + b, ast.Sub: lambda a, b: a - b, ast.Mult: lambda a, b: a * b,
           ast.FloorDiv: lambda a, b: a // b}


def evaluate(expression, env: Mapping[str, int]) -> int:
    """``expression`` may already be an int.  Raises ValidationError on anything outside the
    language, on unknown names, on division by zero and on negative results."""
    if isinstance(expression, bool):
        raise ValidationError("boolean is not an integer expression")
    if isinstance(expression, int):
        value = expression
    elif isinstance(expression, str):
        try:
            tree = ast.parse(expression, mode="eval")
        except SyntaxError as exc:
            raise ValidationError(f"cannot parse expression {expression!r}") from exc
        value = _walk(tree.body, env, expression)
    else:
        raise ValidationError(f"unsupported expression {expression!r}")
    if value < 0:
        raise ValidationError(f"expression {expression!r} evaluates to a negative number")
    return value


def _walk(node: ast.AST, env: Mapping[str, int], source: str) -> int:
    if isinstance(node, ast.Constant) and isinstance(node.value, int) and not isinstance(node.value, bool):
        return node.value
    if isinstance(node, ast.Name):
        if node.id not in env:
            raise ValidationError(f"unknown name {node.id!r} in expression {source!r}")
        return int(env[node.id])
    if isinstance(node, ast.BinOp) and type(node.op) in _BINARY:
        left, right = _walk(node.left, env, source), _walk(node.right, env, source)
        if isinstance(node.op, ast.FloorDiv) and right == 0:
            raise ValidationError(f"division by zero in expression {source!r}")
        return _BINARY[type(node.op)](left, right)
    if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in _FUNCTIONS and not node.keywords:
        args = [_walk(a, env, source) for a in node.args]
        if len(args) != 2 or (node.func.id in ("ceil_div", "align") and args[1] <= 0):
            raise ValidationError(f"bad call in expression {source!r}")
        return _FUNCTIONS[node.func.id](*args)
    raise ValidationError(f"expression {source!r} uses an unsupported construct")
