"""Typed re-exports of the native extension's classes."""
