"""Recipes are scripts launched by ``tune run``; they are not an importable library
(parity: recipes/__init__.py of the reference raises on import for the same reason)."""
raise ModuleNotFoundError(
    "The recipes directory holds entry-point scripts, not a Python package. "
    "Launch them with `tune run <recipe> --config <config>` or copy them with `tune cp`."
)
