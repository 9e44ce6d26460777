"""Computer-aided-engineering metrics."""
