"""Weather / climate metrics and losses."""
