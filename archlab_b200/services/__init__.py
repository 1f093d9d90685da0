"""Side systems kept out of the hot path: metric ledgers, storage hygiene, a chat front, rewards, reports."""
