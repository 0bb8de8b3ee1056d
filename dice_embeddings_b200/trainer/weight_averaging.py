"""Weight-averaging callbacks (filled in below)."""
