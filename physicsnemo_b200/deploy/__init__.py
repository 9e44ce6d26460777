"""Deployment helpers."""
