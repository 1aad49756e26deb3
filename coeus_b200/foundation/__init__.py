"""Foundation layer: error model, core types, memory utilities and iterator adapters
(the counterpart of ``src/foundation/`` in the reference)."""
