"""Small helpers shared by the Python layers (math, logging, torch glue)."""
